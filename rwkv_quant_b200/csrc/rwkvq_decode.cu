// Every kernel here may be launched programmatically (resident while its producer is
// still running), so values produced by earlier kernels are read with L2-coherent
// loads (__ldcg) after pdl_wait(); only weights and parameters use cached paths.
//
// Single-token decode step of a quantized RWKV-7 model: the glue kernels between
// the GEMVs and the host-side launch sequence (rwkvq_decode_step).
//
// Per layer (backends/metal/quant_model.py:638-728, 803-836):
//   ln_shift_mix   LN1 + token shift + the six lerps           -> xs[6][B][D]
//   gemv x3        r, k, v projections (one fused launch)
//   lora_down      the LoRA down projections w1, a1, v1, g1 as row-chunk partial sums
//   lora_up        activation (tanh / - / - / sigmoid) and the up projections w2, a2, v2, g2
//   tmix_core      decay, gates, kk, k and v updates, WKV-7 step on the 64x64 state,
//                  group norm, bonus, gate                      -> og[B][D]
//   gemv + add     output projection and residual
//   ln_shift_mix   LN2 + token shift + lerp                     -> xk[B][D]
//   gemv + relu^2  ffn key;  gemv + add  ffn value and residual
#include <stdlib.h>

#include <map>
#include <mutex>
#include <utility>

#include "rwkvq_decode_parts.cuh"

namespace rwkvq {

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

// Columns [32 g, 32 g + 32) of row R of an sb6 or sym table as exact fp32 values (the arithmetic of
// decode_element: separate multiply and add), with every load of the group issued before any use:
// 16 bytes of codes, the plane words, the scale record.  Requires 32 | cols and the natural alignment
// of the file buffers (rows of codes are multiples of 16 bytes).
__device__ __forceinline__ void decode_group32(const QView& t, size_t R, int g, float* out) {
    if (t.kind == RWKVQ_KIND_SB6) {
        const int nsb = t.cols >> 8, sbi = g >> 3, j = g & 7;
        const uint4 cw = *reinterpret_cast<const uint4*>(t.codes + R * (t.cols >> 1) + g * 16);
        const uint32_t h1 = t.qh ? *reinterpret_cast<const uint32_t*>(t.qh + R * (t.cols >> 3) + g * 4) : 0u;
        const uint32_t h2 = t.qh2 ? *reinterpret_cast<const uint32_t*>(t.qh2 + R * (t.cols >> 3) + g * 4) : 0u;
        const uint32_t* mp = reinterpret_cast<const uint32_t*>(t.qsqm + (R * nsb + sbi) * 12);
        const uint32_t m0 = mp[0], m1 = mp[1], m2 = mp[2];
        const float d = __half2float(t.d[R * nsb + sbi]), dm = __half2float(t.dm[R * nsb + sbi]);
        float sc, mn;
        sb6_scale_min(m0, m1, m2, j, d, dm, sc, mn);
        const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
        for (int k = 0; k < 16; ++k) {               // byte k: column k (low nibble), column k + 16 (high nibble)
            const uint32_t byte = (w[k >> 2] >> (8 * (k & 3))) & 0xFFu;
            const uint32_t lo = (byte & 0xFu) + 16u * ((h1 >> k) & 1u) + 32u * ((h2 >> k) & 1u);
            const uint32_t hi = (byte >> 4) + 16u * ((h1 >> (k + 16)) & 1u) + 32u * ((h2 >> (k + 16)) & 1u);
            out[k] = __fadd_rn(__fmul_rn(static_cast<float>(lo), sc), mn);
            out[k + 16] = __fadd_rn(__fmul_rn(static_cast<float>(hi), sc), mn);
        }
    } else {                                         // sym: two blocks of 16
        const int nb = t.cols >> 4, nsb = t.cols >> 8;
        const float d = __half2float(t.d[R * nsb + (g >> 3)]);
        const uint32_t qs2 = *reinterpret_cast<const unsigned short*>(t.qs + R * nb + 2 * g);
        float s[2];
#pragma unroll
        for (int b2 = 0; b2 < 2; ++b2)
            s[b2] = half_roundtrip(__fmul_rn(static_cast<float>(static_cast<int8_t>((qs2 >> (8 * b2)) & 0xFFu)), d));
        if (t.bits == 8) {
            const uint4* cp = reinterpret_cast<const uint4*>(t.codes + R * t.cols + g * 32);
            const uint4 c0 = cp[0], c1 = cp[1];
            const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
            for (int k = 0; k < 32; ++k)
                out[k] = __fmul_rn(static_cast<float>(static_cast<int8_t>((w[k >> 2] >> (8 * (k & 3))) & 0xFFu)), s[k >> 4]);
        } else {
            const uint4 cw = *reinterpret_cast<const uint4*>(t.codes + R * (t.cols >> 1) + g * 16);
            const uint32_t h1 = t.qh ? *reinterpret_cast<const uint32_t*>(t.qh + R * (t.cols >> 3) + g * 4) : 0u;
            const uint32_t h2 = t.qh2 ? *reinterpret_cast<const uint32_t*>(t.qh2 + R * (t.cols >> 3) + g * 4) : 0u;
            const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
            for (int b2 = 0; b2 < 2; ++b2)
#pragma unroll
                for (int k = 0; k < 8; ++k) {        // block b2, byte k: column k (low nibble), column k + 8 (high nibble)
                    const uint32_t byte = (w[2 * b2 + (k >> 2)] >> (8 * (k & 3))) & 0xFFu;
                    const int c_lo = 16 * b2 + k, c_hi = c_lo + 8;
                    const int lo = static_cast<int>((byte & 0xFu) + 16u * ((h1 >> c_lo) & 1u) + 32u * ((h2 >> c_lo) & 1u)) - 32;
                    const int hi = static_cast<int>((byte >> 4) + 16u * ((h1 >> c_hi) & 1u) + 32u * ((h2 >> c_hi) & 1u)) - 32;
                    out[c_lo] = __fmul_rn(static_cast<float>(lo), s[b2]);
                    out[c_hi] = __fmul_rn(static_cast<float>(hi), s[b2]);
                }
        }
    }
}
__device__ __forceinline__ bool group32_ok(const QView& t) {
    if (t.cols % 256 != 0) return false;
    if (t.kind == RWKVQ_KIND_SB6) return t.gs == 32 && t.sb == 8;
    return t.kind == RWKVQ_KIND_SYM && t.gs == 16 && t.sb == 16;
}

// x[b] = LN0(fp16(bf16(dequant(emb[token[b]])))): one embedding row is decoded from the
// packed table (quant_model.py:853, 975-976; rounding policy :128-154).  sb6 / sym tables: one
// thread per 32 columns decodes its group with all loads in flight at once and hands the row over
// through shared memory; other layouts: element by element.
__global__ void __launch_bounds__(kRowThreads) embed_ln0_kernel(QView emb, const long long* tokens,
                                                               const float* ln_w, const float* ln_b,
                                                               float* x, int D) {
    __shared__ float red[kRowThreads / 32];
    __shared__ float srow[kRowThreads * kRowPer];
    const int b = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    long long tok = __ldcg(tokens + b);
    tok = tok < 0 ? 0 : (tok >= emb.rows ? emb.rows - 1 : tok);
    float v[kRowPer];
    if (group32_ok(emb)) {
        for (int g = threadIdx.x; g < D / 32; g += kRowThreads) {
            float o[32];
            decode_group32(emb, static_cast<size_t>(tok), g, o);
#pragma unroll
            for (int k = 0; k < 32; ++k) srow[g * 32 + k] = dense_param_rounding(o[k]);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kRowPer; ++i) {
            const int d = threadIdx.x + i * kRowThreads;
            v[i] = (d < D) ? srow[d] : 0.f;
        }
    } else {
#pragma unroll
        for (int i = 0; i < kRowPer; ++i) {
            const int d = threadIdx.x + i * kRowThreads;
            v[i] = (d < D) ? dense_param_rounding(decode_element(emb, static_cast<int>(tok), d)) : 0.f;
        }
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
// All loads are issued before the reductions so that their latencies overlap.  PER: elements per
// thread (8 serves D <= 2048 and leaves registers for the lerp vectors, which are then loaded with the
// LayerNorm parameters before the launch wait; 16 serves D <= 4096 and reads them where they are used).
template <int NMIX, int PER>
__global__ void __launch_bounds__(kRowThreads) ln_shift_mix_kernel(const float* __restrict__ x,
                                                                  const float* __restrict__ ln_w,
                                                                  const float* __restrict__ ln_b,
                                                                  float* __restrict__ shift,
                                                                  const float* __restrict__ mix,
                                                                  float* __restrict__ out, int B, int D,
                                                                  __half* __restrict__ x16_out, __half* __restrict__ x16lo_out,
                                                                  __half* __restrict__ xsum_out,
                                                                  float* __restrict__ unscale_out, int x16_mask,
                                                                  float* __restrict__ zero_a, float* __restrict__ zero_b) {
    // x16_out (optional) [max(NMIX, 1)][B][D] with unscale_out [max(NMIX, 1)][B]: the rows selected by
    // x16_mask also as fp16(out * 2^s), s chosen from the row's max so that no value leaves the fp16
    // range, and 2^-s: the form the single-term small-batch linear reads (half the bytes, no
    // conversion there); x16lo_out with xsum_out (optional; D a multiple of 128): the form the two-term
    // tcgen05 linear reads: s is then chosen for |out * 2^s| <= 2^9, x16lo_out (same shape) takes
    // fp16(out * 2^s - x16_out) and xsum_out [max(NMIX, 1)][B][D / 128][8] the sums of out * 2^s over the
    // four 32-column blocks of every 128 columns, 4 high halves then 4 low halves.  With unscale_out
    // alone, max|out| of the selected rows goes there instead (what the two-term mma.sync linear wants
    // beside the fp32 rows);
    // zero_a / zero_b (optional) [B]: slots later kernels of the layer merge their own row maxima
    // into, cleared here for stream b
    constexpr int NM = NMIX > 0 ? NMIX : 1;
    __shared__ float red[kRowThreads / 32];
    __shared__ float redm[kRowThreads / 32][NM];
    const int b = blockIdx.x;
    float v[PER], prev[PER], lw[PER], lb[PER];
    constexpr bool PRE = PER <= 8 && NMIX > 0;              // lerp vectors in registers
    float mxr[PRE ? NMIX : 1][PRE ? PER : 1];
    pdl_launch_dependents();
#pragma unroll
    for (int i = 0; i < PER; ++i) {          // parameters do not depend on the previous kernel
        const int d = threadIdx.x + i * kRowThreads;
        lw[i] = d < D ? ln_w[d] : 0.f;
        lb[i] = d < D ? ln_b[d] : 0.f;
        if (PRE) {
#pragma unroll
            for (int m = 0; m < NMIX; ++m) mxr[PRE ? m : 0][PRE ? i : 0] = d < D ? __ldg(mix + m * D + d) : 0.f;
        }
    }
    pdl_wait();
    if (threadIdx.x == 0) {
        if (zero_a) zero_a[b] = 0.f;
        if (zero_b) zero_b[b] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = threadIdx.x + i * kRowThreads;
        const bool ok = d < D;
        const size_t bd = static_cast<size_t>(b) * D + d;
        v[i] = ok ? __ldcg(x + bd) : 0.f;
        prev[i] = (ok && NMIX > 0) ? __ldcg(shift + bd) : 0.f;
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) s += v[i];
    const float mean = block_sum(s, red) / D;
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const float c = (threadIdx.x + i * kRowThreads < D) ? v[i] - mean : 0.f;
        s2 += c * c;
    }
    const float inv = 1.0f / sqrtf(block_sum(s2, red) / D + 1e-5f);
    float mx[NM];
#pragma unroll
    for (int m = 0; m < NM; ++m) mx[m] = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = threadIdx.x + i * kRowThreads;
        if (d >= D) continue;
        const size_t bd = static_cast<size_t>(b) * D + d;
        const float xn = (v[i] - mean) * inv * lw[i] + lb[i];
        if (NMIX == 0) { out[bd] = xn; mx[0] = fmaxf(mx[0], fabsf(xn)); continue; }
        const float xx = prev[i] - xn;
        shift[bd] = xn;
#pragma unroll
        for (int m = 0; m < NMIX; ++m) {
            const float o = xn + xx * (PRE ? mxr[PRE ? m : 0][PRE ? i : 0] : __ldg(mix + m * D + d));
            out[(static_cast<size_t>(m) * B) * D + bd] = o;
            mx[m < NM ? m : 0] = fmaxf(mx[m < NM ? m : 0], fabsf(o));
        }
    }
    if (unscale_out != nullptr) {
        __shared__ float sc_m[NM];
#pragma unroll
        for (int m = 0; m < NM; ++m) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx[m] = fmaxf(mx[m], __shfl_xor_sync(0xFFFFFFFFu, mx[m], o));
            if ((threadIdx.x & 31) == 0) redm[threadIdx.x >> 5][m] = mx[m];
        }
        __syncthreads();
        if (threadIdx.x < NM) {
            float r = 0.f;
            for (int w = 0; w < kRowThreads / 32; ++w) r = fmaxf(r, redm[w][threadIdx.x]);
            if (x16_out == nullptr) {
                if ((x16_mask >> threadIdx.x) & 1) unscale_out[threadIdx.x * B + b] = r;
                return;
            }
            // |x| * 2^(14 - e) <= 2^14 with max|x| <= 2^e (2^9 for the two-term form, whose block sums must
            // stay inside the fp16 range); a non-finite row keeps scale 1 and propagates
            float s1 = 1.f, u1 = 1.f;
            if (r > 0.f && r < INFINITY) {
                int e = 0;
                frexpf(r, &e);
                e = max(-100, e);
                const int top = x16lo_out ? 9 : 14;
                s1 = ldexpf(1.f, top - e);
                u1 = ldexpf(1.f, e - top);
            }
            sc_m[threadIdx.x] = s1;
            if ((x16_mask >> threadIdx.x) & 1) unscale_out[threadIdx.x * B + b] = u1;
        }
        if (x16_out == nullptr) return;
        __syncthreads();
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = threadIdx.x + i * kRowThreads;
            if (d >= D) continue;
            const size_t bd = static_cast<size_t>(b) * D + d;
            const float xn = (v[i] - mean) * inv * lw[i] + lb[i];
            // d >= D holds for a whole warp or for none of it (D is a multiple of 32 whenever xsum_out is given)
            auto emit = [&](int m, float sx) {
                const size_t o = (static_cast<size_t>(m) * B) * D + bd;
                const __half hi = __float2half_rn(sx);
                x16_out[o] = hi;
                if (x16lo_out == nullptr) return;
                x16lo_out[o] = __float2half_rn(sx - __half2float(hi));
                float bs = sx;                                   // the warp holds one block of 32 columns
#pragma unroll
                for (int sh = 16; sh > 0; sh >>= 1) bs += __shfl_xor_sync(0xFFFFFFFFu, bs, sh);
                if ((threadIdx.x & 31) == 0) {
                    const int blk = d >> 5;
                    __half* sp = xsum_out + ((static_cast<size_t>(m) * B + b) * (D >> 7) + (blk >> 2)) * 8 + (blk & 3);
                    const __half sh16 = __float2half_rn(bs);
                    sp[0] = sh16;
                    sp[4] = __float2half_rn(bs - __half2float(sh16));
                }
            };
            if (NMIX == 0) { emit(0, xn * sc_m[0]); continue; }
            const float xx = prev[i] - xn;
#pragma unroll
            for (int m = 0; m < NMIX; ++m) {
                if (!((x16_mask >> m) & 1)) continue;
                const float o = xn + xx * (PRE ? mxr[PRE ? m : 0][PRE ? i : 0] : __ldg(mix + m * D + d));
                emit(m, o * sc_m[m < NM ? m : 0]);
            }
        }
    }
}

// ---- batched LoRA products, tensors stored [in, out] (a warp reads 128 contiguous codes)
//
// down:  part[br][chunk][n][j] = sum_{i in chunk} x_br[n][i] * W1_br[i][j]     (j < rank)
//        grid (row chunks of 64, branches); the partial sums go to scratch in a fixed
//        layout and are added in chunk order by the consumer, so the result does not
//        depend on scheduling.
// up:    h[j] = act_br(sum_chunk part[br][chunk][n][j]);  y_br[n][c] = sum_j h[j] * W2_br[j][c]
//        grid (column tiles of 128, branches).
constexpr int kLmMaxN = 8;            // right-hand sides per launch
constexpr int kLdRows = 64;           // rows of W1 per CTA
constexpr int kLuCols = 128;          // columns of W2 per CTA
constexpr int kLmMaxRank = 512;

struct LoraDownArgs {
    QView t[4];
    const float* x[4];      // [n_cols, ldx]
    float* part;            // [4][n_chunks][n_stride][max_rank]
    long long ldx;
    int n_cols, n_chunks, max_rank;
    int n_stride;           // right-hand sides the scratch is laid out for (multiple of kLmMaxN)
    int rep;                // 64-row sub-chunks one CTA accumulates (more for large batches: fewer partial sums)
};
struct LoraUpArgs {
    QView t[4];
    const float* part;
    float* y[4];            // [n_cols, ldy]
    int act[4];
    long long ldy;
    int n_cols, n_chunks, max_rank, n_stride;
};

// 256 threads = 4 row groups x 64 column threads (4 columns each, 256 columns per pass)
// MULTI = false: one 64-row chunk per CTA (the batch-1 form, loops resolved at compile time)
template <int MODE, bool MULTI>
__device__ __forceinline__ void lora_down_body(const LoraDownArgs& a, const QView& t, const float* __restrict__ xall,
                                               float (&red)[4][kLmMaxN][256]) {
    const int chunk = blockIdx.x, br = blockIdx.y;
    const int n0 = blockIdx.z * kLmMaxN;                  // this CTA's group of right-hand sides
    const int nc = min(kLmMaxN, a.n_cols - n0);
    const float* x = xall + static_cast<size_t>(n0) * a.ldx;
    const int rg = threadIdx.x >> 6, ct = threadIdx.x & 63;
    const int nb = MODE == 0 ? (t.cols + t.gs - 1) / t.gs : 0;
    for (int c0 = 0; c0 < t.cols; c0 += 256) {
        const int c = c0 + ct * 4;
        const int blk = MODE == 0 ? c / t.gs : 0;
        float acc[kLmMaxN][4];
#pragma unroll
        for (int n = 0; n < kLmMaxN; ++n)
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[n][k] = 0.f;
        const int rep = MULTI ? a.rep : 1;
#pragma unroll 1
        for (int sub = 0; sub < rep; ++sub) {
            const int row0 = (chunk * rep + sub) * kLdRows;
            if (c < t.cols && row0 < t.rows) {
                constexpr int RPT = kLdRows / 4;          // rows per thread, all loads issued together
                float w[RPT][4];
#pragma unroll
                for (int r = 0; r < RPT; ++r) lora_w4<MODE>(t, min(row0 + rg + 4 * r, t.rows - 1), c, nb, blk, w[r]);
                pdl_wait();              // the weights above are constants; x comes from the previous kernel
#pragma unroll
                for (int n = 0; n < kLmMaxN; ++n) {
                    if (n >= nc) break;
#pragma unroll
                    for (int r = 0; r < RPT; ++r) {
                        const int i = row0 + rg + 4 * r;
                        const float xv = i < t.rows ? __ldcg(x + n * a.ldx + i) : 0.f;
#pragma unroll
                        for (int k = 0; k < 4; ++k) acc[n][k] = fmaf(xv, w[r][k], acc[n][k]);
                    }
                }
            }
        }
        pdl_wait();
        __syncthreads();
#pragma unroll
        for (int n = 0; n < kLmMaxN; ++n) {
            if (n >= nc) break;
#pragma unroll
            for (int k = 0; k < 4; ++k) red[rg][n][ct * 4 + k] = acc[n][k];
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < nc * 256; idx += 256) {
            const int n = idx >> 8, cc = idx & 255;
            if (c0 + cc >= t.cols) continue;
            const float v = (red[0][n][cc] + red[1][n][cc]) + (red[2][n][cc] + red[3][n][cc]);
            a.part[((static_cast<size_t>(br) * a.n_chunks + chunk) * a.n_stride + n0 + n) * a.max_rank + c0 + cc] = v;
        }
    }
}

template <bool MULTI>
__global__ void __launch_bounds__(256) lora_down_kernel(const LoraDownArgs a) {
    __shared__ float red[4][kLmMaxN][256];
    const QView& t = a.t[blockIdx.y];
    const float* x = a.x[blockIdx.y];
    pdl_launch_dependents();
    switch (lora_mode(t)) {
        case 0: lora_down_body<0, MULTI>(a, t, x, red); break;
        case 1: lora_down_body<1, MULTI>(a, t, x, red); break;
        default: lora_down_body<2, MULTI>(a, t, x, red); break;
    }
}

// 256 threads = 8 row groups x 32 column threads (4 columns each)
template <int MODE>
__device__ __forceinline__ void lora_up_body(const LoraUpArgs& a, int n_cols, const QView& t,
                                             const float (&h)[kLmMaxN][kLmMaxRank], float (&acc)[kLmMaxN][4]) {
    const int rg = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * kLuCols + lane * 4;
    const int rank = t.rows;
    const int nb = MODE == 0 ? (t.cols + t.gs - 1) / t.gs : 0;
    const int blk = MODE == 0 ? c / t.gs : 0;
    if (c >= t.cols) return;
    for (int j0 = rg; j0 < rank; j0 += 64) {          // 8 rows of this thread per batch of loads
        float w[8][4];
#pragma unroll
        for (int r = 0; r < 8; ++r) lora_w4<MODE>(t, min(j0 + 8 * r, rank - 1), c, nb, blk, w[r]);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const int j = j0 + 8 * r;
            if (j >= rank) break;
#pragma unroll
            for (int n = 0; n < kLmMaxN; ++n) {
                if (n >= n_cols) break;
                const float hv = h[n][j];
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[n][k] = fmaf(hv, w[r][k], acc[n][k]);
            }
        }
    }
}

__global__ void __launch_bounds__(256) lora_up_kernel(const LoraUpArgs a) {
    __shared__ float h[kLmMaxN][kLmMaxRank];
    __shared__ float red[8][kLmMaxN][kLuCols];
    const int br = blockIdx.y;
    const QView& t = a.t[br];
    pdl_launch_dependents();
    pdl_wait();
    if (blockIdx.x * kLuCols >= t.cols) return;
    const int rank = t.rows;
    const int n0 = blockIdx.z * kLmMaxN;                      // this CTA's group of right-hand sides
    const int nc = min(kLmMaxN, a.n_cols - n0);
    for (int idx = threadIdx.x; idx < nc * rank; idx += 256) {
        const int n = idx / rank, j = idx % rank;
        const float* pp = a.part + ((static_cast<size_t>(br) * a.n_chunks) * a.n_stride + n0 + n) * a.max_rank + j;
        const size_t stride = static_cast<size_t>(a.n_stride) * a.max_rank;
        float v = 0.f;
        int ch = 0;
        for (; ch + 8 <= a.n_chunks; ch += 8) {       // 8 loads in flight, summed in chunk order
            float pv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) pv[u] = __ldcg(pp + (ch + u) * stride);
#pragma unroll
            for (int u = 0; u < 8; ++u) v += pv[u];
        }
        for (; ch < a.n_chunks; ++ch) v += __ldcg(pp + ch * stride);
        if (a.act[br] == 1) v = tanhf(v);
        else if (a.act[br] == 2) v = sigmoidf_(v);
        h[n][j] = v;
    }
    __syncthreads();
    const int rg = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float acc[kLmMaxN][4];
#pragma unroll
    for (int n = 0; n < kLmMaxN; ++n)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[n][k] = 0.f;
    switch (lora_mode(t)) {
        case 0: lora_up_body<0>(a, nc, t, h, acc); break;
        case 1: lora_up_body<1>(a, nc, t, h, acc); break;
        default: lora_up_body<2>(a, nc, t, h, acc); break;
    }
#pragma unroll
    for (int n = 0; n < kLmMaxN; ++n) {
        if (n >= nc) break;
#pragma unroll
        for (int k = 0; k < 4; ++k) red[rg][n][lane * 4 + k] = acc[n][k];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nc * kLuCols; idx += 256) {
        const int n = idx / kLuCols, cc = idx % kLuCols;
        const int col = blockIdx.x * kLuCols + cc;
        if (col >= t.cols) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += red[w][n][cc];
        a.y[br][static_cast<size_t>(n0 + n) * a.ldy + col] = v;
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
    float* og_amax;                    // optional [B]: max|og| per stream is merged into it (atomic max on the bits)
};

// sum over 64 shared-memory values, computed redundantly by every warp (two values per lane):
// no block-wide barrier beyond the one that published the values
__device__ __forceinline__ float warp_sum64(const float* v, int lane) {
    float s = v[lane] + v[lane + 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    return s;
}

__global__ void __launch_bounds__(256) tmix_core_kernel(const TmixCoreArgs p) {
    // per-column operands of the state update, written once by warps 0 and 1 and read as float4 by all:
    // sA = -kk / |kk|, sB = (kk / |kk|) * a_gate, sW decay, sK key, sR receptance
    __shared__ __align__(16) float sA[64], sB[64], sW[64], sK[64], sR[64];
    __shared__ float sV[64], sY[64], sG[64], sT[64];
    const int hi = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
    const size_t row = static_cast<size_t>(b) * p.D + hi * 64;
    // the state slice of this thread is requested first: it is the largest load
    // thread (dv, part) owns columns 16 i + 4 part + e of state row dv (i, e < 4): every load
    // instruction of a quad covers 64 contiguous bytes
    const int dv = tid >> 2, part = tid & 3;
    float* hp = p.state + ((static_cast<size_t>(b) * p.H + hi) * 64 + dv) * 64 + part * 4;
    float h[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 v4 = __ldcs(reinterpret_cast<const float4*>(hp + 16 * i));
        h[4 * i] = v4.x; h[4 * i + 1] = v4.y; h[4 * i + 2] = v4.z; h[4 * i + 3] = v4.w;
    }
    pdl_launch_dependents();
    // per-channel parameters of warps 0 and 1 (channel hi * 64 + tid; r_k also for the partner channel of the
    // final dot product): nothing the kernels before this one write, so they are loaded before the wait
    float pw0 = 0.f, pa0 = 0.f, pka = 0.f, pkk = 0.f, pv0 = 0.f, prk0 = 0.f, prk1 = 0.f, plw = 0.f, plb = 0.f;
    if (tid < 64) {
        const int c = hi * 64 + tid;
        pw0 = __ldg(p.w0 + c); pa0 = __ldg(p.a0 + c); pka = __ldg(p.k_a + c); pkk = __ldg(p.k_k + c);
        if (!p.layer0) pv0 = __ldg(p.v0 + c);
        prk0 = __ldg(p.r_k + hi * 64 + lane); prk1 = __ldg(p.r_k + hi * 64 + lane + 32);
        plw = __ldg(p.lnx_w + c); plb = __ldg(p.lnx_b + c);
    }
    pdl_wait();            // the state above was written a whole token ago
    if (tid < 64) {
        const float r = __ldcg(p.r + row + tid), k = __ldcg(p.k + row + tid);
        float v = __ldcg(p.v + row + tid);
        const float w = expf(-0.606531f * sigmoidf_(__ldcg(p.yw + row + tid) + pw0));
        const float av = sigmoidf_(__ldcg(p.ya + row + tid) + pa0);
        const float k2 = k * (1.0f + (av - 1.0f) * pka);
        if (p.layer0) p.v_first[row + tid] = v;
        else v = v + (__ldcg(p.v_first + row + tid) - v) * sigmoidf_(__ldcg(p.yv + row + tid) + pv0);
        const float kk = k * pkk;
        sT[tid] = kk * kk;
        sW[tid] = w; sK[tid] = k2; sR[tid] = r; sV[tid] = v; sG[tid] = __ldcg(p.g + row + tid);
        asm volatile("bar.sync 1, 64;" ::: "memory");        // warps 0 and 1 only: sT is complete
        // both warps reduce the head-wide sum themselves; a = -kk / |kk|, b = -a * a_gate
        const float kn = kk * (1.0f / sqrtf(warp_sum64(sT, lane) + 1e-12f));
        sA[tid] = -kn;
        sB[tid] = kn * av;
    }
    __syncthreads();
    // one WKV-7 step on the thread's 16 state columns
    float sa = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 a4 = *reinterpret_cast<const float4*>(sA + 16 * i + 4 * part);
        sa = fmaf(h[4 * i], a4.x, sa); sa = fmaf(h[4 * i + 1], a4.y, sa);
        sa = fmaf(h[4 * i + 2], a4.z, sa); sa = fmaf(h[4 * i + 3], a4.w, sa);
    }
    sa += __shfl_xor_sync(0xFFFFFFFFu, sa, 1);
    sa += __shfl_xor_sync(0xFFFFFFFFu, sa, 2);
    const float vv = sV[dv];
    float y = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int dk = 16 * i + 4 * part;
        const float4 b4 = *reinterpret_cast<const float4*>(sB + dk), w4 = *reinterpret_cast<const float4*>(sW + dk);
        const float4 k4 = *reinterpret_cast<const float4*>(sK + dk), r4 = *reinterpret_cast<const float4*>(sR + dk);
        h[4 * i] = fmaf(w4.x, h[4 * i], fmaf(vv, k4.x, sa * b4.x));
        y = fmaf(h[4 * i], r4.x, y);
        h[4 * i + 1] = fmaf(w4.y, h[4 * i + 1], fmaf(vv, k4.y, sa * b4.y));
        y = fmaf(h[4 * i + 1], r4.y, y);
        h[4 * i + 2] = fmaf(w4.z, h[4 * i + 2], fmaf(vv, k4.z, sa * b4.z));
        y = fmaf(h[4 * i + 2], r4.z, y);
        h[4 * i + 3] = fmaf(w4.w, h[4 * i + 3], fmaf(vv, k4.w, sa * b4.w));
        y = fmaf(h[4 * i + 3], r4.w, y);
    }
    y += __shfl_xor_sync(0xFFFFFFFFu, y, 1);
    y += __shfl_xor_sync(0xFFFFFFFFu, y, 2);
#pragma unroll
    for (int i = 0; i < 4; ++i)
        *reinterpret_cast<float4*>(hp + 16 * i) = make_float4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
    if (part == 0) sY[dv] = y;
    __syncthreads();
    if (tid < 64) {            // warps 0 and 1: group norm over the head (two-pass), bonus, gate
        const float mean = warp_sum64(sY, lane) / 64.f;
        const float d0 = sY[lane] - mean, d1 = sY[lane + 32] - mean;
        float var = d0 * d0 + d1 * d1, dp = sR[lane] * sK[lane] * prk0 + sR[lane + 32] * sK[lane + 32] * prk1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            var += __shfl_xor_sync(0xFFFFFFFFu, var, o);
            dp += __shfl_xor_sync(0xFFFFFFFFu, dp, o);
        }
        const float nrm = (sY[tid] - mean) * (1.0f / sqrtf(var / 64.f + 64e-5f));
        const float o = (nrm * plw + plb + dp * sV[tid]) * sG[tid];
        p.og[row + tid] = o;
        if (p.og_amax != nullptr) {          // warps 0 and 1 hold the 64 outputs
            float m = fabsf(o);
#pragma unroll
            for (int of = 16; of > 0; of >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, of));
            if ((tid & 31) == 0) atomicMax(reinterpret_cast<int*>(p.og_amax) + b, __float_as_int(m));
        }
    }
}

// greedy argmax in two stages (lowest index wins ties): 64 slices per row, then one CTA
constexpr int kArgSlices = 64;
__global__ void __launch_bounds__(256) argmax_partial_kernel(const float* logits, float* pv, int* pi, int V) {
    __shared__ float bv[8];
    __shared__ int bi[8];
    pdl_launch_dependents();
    pdl_wait();
    const float* row = logits + static_cast<size_t>(blockIdx.y) * V;
    const int per = (V + kArgSlices - 1) / kArgSlices;
    const int lo = blockIdx.x * per, hi = min(lo + per, V);
    float best = -INFINITY;
    int idx = V;
    for (int i = lo + threadIdx.x; i < hi; i += 256) argmax_combine(best, idx, __ldcg(row + i), i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        argmax_combine(best, idx, __shfl_xor_sync(0xFFFFFFFFu, best, o), __shfl_xor_sync(0xFFFFFFFFu, idx, o));
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) argmax_combine(best, idx, bv[w], bi[w]);
        pv[blockIdx.y * kArgSlices + blockIdx.x] = best;
        pi[blockIdx.y * kArgSlices + blockIdx.x] = idx;
    }
}
__global__ void __launch_bounds__(kArgSlices) argmax_final_kernel(const float* pv, const int* pi, long long* out, int V) {
    pdl_wait();
    float best = __ldcg(pv + blockIdx.x * kArgSlices + threadIdx.x);
    int idx = __ldcg(pi + blockIdx.x * kArgSlices + threadIdx.x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        argmax_combine(best, idx, __shfl_xor_sync(0xFFFFFFFFu, best, o), __shfl_xor_sync(0xFFFFFFFFu, idx, o));
    __shared__ float bv[2];
    __shared__ int bi[2];
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        argmax_combine(best, idx, bv[1], bi[1]);
        out[blockIdx.x] = idx < V ? idx : 0;
    }
}

}  // namespace rwkvq

using namespace rwkvq;

namespace {

constexpr int kBatchMax = 256;     // streams up to which the small-batch kernel serves the linears of a step
inline bool batch_path(int B) { return B > 2 && B <= kBatchMax; }
// Which small-batch kernel: measured on B200 (1.5B, whole decode step) the tcgen05 form wins from 33
// streams on (64 streams: 3.77 against 4.43 ms per step) and loses below (32: 2.87 / 2.68 ms, 8: 2.42 / 2.01 ms):
// its pass (dependent weight loads -> conversion -> MMA) is longer than a warp-iteration of the mma.sync form
inline bool tcb_pays(int B) { return batch_fast() && tcb_enabled() && B > 32; }
// Default (two-term) precision above 32 streams: which linears run on the tcgen05 form of the two-term
// kernel, fed with fp16 pairs and block sums by the LayerNorm kernels (bit 0 r / k / v, bit 1 ffn key,
// bit 2 head).  The output projection and the ffn value, whose inputs reach the linear as fp32 rows without
// a known scale, always stay on the mma.sync form.  Measured on B200 (1.5B, whole decode step, ms):
//   streams        33    36    40    48    50    52    56    60    64
//   all mma.sync  3.69  3.72  3.72  3.76  3.92  4.02  4.10  4.13  4.05
//   head          3.66  3.69  3.72  3.73   -    3.96  4.04  4.07  4.00
//   r/k/v + head   -    3.70  3.82  3.86  3.80  3.79  3.87  3.92  3.92
//   all three     3.45  3.47  3.59  3.64  4.14  4.20  4.27  4.32  4.27
// -> all three up to 48 streams, r / k / v and the head from 49 to 64.
// RWKVQ_TCB_EXACT in the environment (read once) overrides: 0 none, 1 all three at every such batch.
int g_tcb_exact = -2;          // -2 environment not read yet, -1 the measured policy, 0 none, 1 all three
inline int tcx_mask(int B) {
    if (g_tcb_exact == -2) {
        const char* e = getenv("RWKVQ_TCB_EXACT");
        g_tcb_exact = (e == nullptr || (e[0] != '0' && e[0] != '1')) ? -1 : e[0] - '0';
    }
    if (batch_fast() || !tcb_enabled() || B <= 32 || B > kBatchMax || g_tcb_exact == 0) return 0;
    if (g_tcb_exact == 1) return 7;
    return B <= 48 ? 7 : B <= 64 ? 5 : 0;
}


struct Workspace {
    float *x, *xs, *rkv, *part, *yl, *og, *xk, *hffn, *xo, *v_first, *logits, *argv, *gscratch, *gemm_ws;
    int* status;             // first word of the workspace: RWKVQ_E_TIMEOUT if a bounded device-side wait of a step ran out
    float* amax;             // [10][B] per-row scale inverses / maxima for the small-batch linears: 6 mix rows, og, xk, hffn, xo
    __half *xs16, *xk16, *xo16;     // fp16 forms of the mix rows, the channel-mix row and the final row
    __half *xs16lo, *xk16lo, *xo16lo;   // their second terms (two-term tcgen05 linears)
    __half *xs_sum, *xk_sum, *xo_sum;   // ... and block sums, [rows][B][D / 128][8]
    int n_chunks;
    size_t part_floats;
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
    w.status = reinterpret_cast<int*>(take(64));
    w.x = take(b * D); w.xs = take(6 * b * D); w.rkv = take(3 * b * D);
    w.n_chunks = static_cast<int>((D + kLdRows - 1) / kLdRows);
    w.part_floats = 4 * static_cast<size_t>(w.n_chunks) * ((b + kLmMaxN - 1) / kLmMaxN * kLmMaxN) * R;   // upper bound (rep = 1)
    w.part = take(w.part_floats);
    w.yl = take(4 * b * D); w.og = take(b * D); w.xk = take(b * D); w.hffn = take(b * F);
    w.xo = take(b * D); w.v_first = take(b * D); w.logits = take(b * V);
    w.argv = take(2 * b * kArgSlices);
    w.amax = take(10 * b);
    w.xs16 = reinterpret_cast<__half*>(take(3 * b * D));
    w.xk16 = reinterpret_cast<__half*>(take((b * D + 1) / 2));
    w.xo16 = reinterpret_cast<__half*>(take((b * D + 1) / 2));
    w.xs16lo = reinterpret_cast<__half*>(take(3 * b * D));
    w.xk16lo = reinterpret_cast<__half*>(take((b * D + 1) / 2));
    w.xo16lo = reinterpret_cast<__half*>(take((b * D + 1) / 2));
    w.xs_sum = reinterpret_cast<__half*>(take(6 * b * (D / 32 + 4)));
    w.xk_sum = reinterpret_cast<__half*>(take(b * (D / 32 + 4)));
    w.xo_sum = reinterpret_cast<__half*>(take(b * (D / 32 + 4)));
    w.gscratch = take(gemv_mma_scratch_bytes() / sizeof(float));
    w.gemm_ws = take(rwkvq_gemm_workspace_bytes_for(B, static_cast<int>(F > D ? F : D)) / sizeof(float) + 1);
    w.bytes = off;
    return w;
}

// y_br = (act_br(x_br @ W1_br)) @ W2_br for up to 4 branches, B right-hand sides
// One quantized linear for B right-hand sides; the single-vector tensor-core kernel gets
// the K-split scratch, everything else goes through the public entry point.
// x16 / x_scale: the fp16 form of x with its per-row scale inverses (what the LayerNorm kernels write
// on the small-batch path), or null with x_scale = max|x| per row for fp32 rows; x16lo: the second fp16
// term of x, which selects the two-term tcgen05 kernel (the caller has checked gemm_tcb_ok); y_amax:
// optional slots max|y| per row is merged into.
int linear(const rwkvq_qtensor* t, const float* x, int B, int in, float* y, int out, int epi, const float* resid,
           float* scratch, void* gemm_ws, void* stream, const __half* x16 = nullptr, const float* x_scale = nullptr,
           float* y_amax = nullptr, int* status = nullptr, const __half* x16lo = nullptr, const __half* xsum = nullptr) {
    const int ml = mma_layout_of(*t);
    if (B == 1 && ml >= 0) {
        int rc = validate_qtensor(t, "rwkvq_decode_step(linear)");
        if (rc) return rc;
        return launch_gemv_mma(ml, t, 1, x, RWKVQ_F32, in, y, out, epi, resid, 0, static_cast<cudaStream_t>(stream),
                               nullptr, scratch);
    }
    if (batch_path(B) && ml >= 0 && x_scale) {            // small batch: weights read once, tokens as MMA columns
        int rc = validate_qtensor(t, "rwkvq_decode_step(linear)");
        if (rc) return rc;
        const void* xs[1] = {x16 ? static_cast<const void*>(x16) : static_cast<const void*>(x)};
        const float* sc[1] = {x_scale};
        float* ys[1] = {y};
        const float* rs[1] = {resid};
        float* ao[1] = {y_amax};
        if (x16 && x16lo) {
            const void* xl[1] = {x16lo};
            const void* xm[1] = {xsum};
            return launch_gemm_tcb(t, 1, xs, true, sc, B, in, ys, out, epi, rs, ao, status, static_cast<cudaStream_t>(stream), true, xl, xm);
        }
        if (tcb_pays(B) && gemm_tcb_ok(*t))
            return launch_gemm_tcb(t, 1, xs, x16 != nullptr, sc, B, in, ys, out, epi, rs, ao, status, static_cast<cudaStream_t>(stream));
        return launch_gemv_batch(t, 1, xs, x16 != nullptr, sc, B, in, ys, out, epi, rs, ao, static_cast<cudaStream_t>(stream));
    }
    if (B > 2 && (t->kind == RWKVQ_KIND_SB6 || t->kind == RWKVQ_KIND_SYM))     // tcgen05 path for large batches
        return rwkvq_gemm(t, x, B, in, y, out, epi, resid, gemm_ws, rwkvq_gemm_workspace_bytes_for(B, in), stream);
    return rwkvq_gemv(t, x, RWKVQ_F32, B, in, y, out, epi, resid, stream);
}

// The LoRA branches depend on the normalised row only, not on r/k/v: they run on a side
// stream between a fork after LN1 and a join before the time-mix core, so that in a captured
// graph they form a parallel branch beside the r/k/v GEMV instead of two more links of the
// dependent chain.  One side stream and two events per (device, caller stream), created on the
// first call that uses that stream (make it outside stream capture): sequences issued on
// different streams, from one or several host threads, never share an event.  Calls on the SAME
// stream must come from one thread at a time, as for any stream-ordered API.
// RWKVQ_FORK=0 keeps everything on the caller's stream.
struct SideLane { cudaStream_t stream = nullptr; cudaEvent_t fork = nullptr, join = nullptr; };
SideLane* side_lane(cudaStream_t caller) {
    static const bool enabled = [] { const char* e = getenv("RWKVQ_FORK"); return !(e && e[0] == '0'); }();
    if (!enabled) return nullptr;
    static std::mutex mu;
    static std::map<std::pair<int, cudaStream_t>, SideLane> lanes;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    SideLane& l = lanes[std::make_pair(dev, caller)];
    if (!l.stream) {
        SideLane n;
        if (cudaStreamCreateWithFlags(&n.stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&n.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&n.join, cudaEventDisableTiming) != cudaSuccess) {
            if (n.fork) cudaEventDestroy(n.fork);
            if (n.stream) cudaStreamDestroy(n.stream);
            return nullptr;
        }
        l = n;
    }
    return &l;
}

int lora_rep(int B) { return B > kLmMaxN ? 8 : 1; }

int lora_pair(const rwkvq_qtensor* const* t1, const rwkvq_qtensor* const* t2, const float* const* xs,
              float* const* ys, const int* acts, int n_br, int B, int D, int max_rank, float* part,
              size_t part_floats, int n_chunks, cudaStream_t s) {
    LoraDownArgs d{};
    LoraUpArgs u{};
    int max_cols = 0;
    for (int i = 0; i < n_br; ++i) {
        int rc = validate_qtensor(t1[i], "rwkvq_decode_step(lora down)");
        if (rc) return rc;
        rc = validate_qtensor(t2[i], "rwkvq_decode_step(lora up)");
        if (rc) return rc;
        RWKVQ_REQUIRE(t1[i]->rows == D && t1[i]->cols == t2[i]->rows && t1[i]->cols <= max_rank &&
                          t1[i]->cols <= kLmMaxRank,
                      RWKVQ_E_SHAPE, "rwkvq_decode_step: LoRA branch %d has shapes [%d,%d] x [%d,%d]", i,
                      t1[i]->rows, t1[i]->cols, t2[i]->rows, t2[i]->cols);
        d.t[i] = make_view(*t1[i]);
        u.t[i] = make_view(*t2[i]);
        u.act[i] = acts[i];
        if (t2[i]->cols > max_cols) max_cols = t2[i]->cols;
    }
    if (B != 2 && lora_mma_ok(t1, t2, n_br, D)) {
        // both products on the tensor cores, matrices read once.  Measured per token: one stream 1.160 ms here
        // against 1.185 ms on the per-stream kernels below, two streams 1.92 against 1.88 ms: those keep two
        // streams and odd shapes.  (A row's result does not depend on the batch it is computed in, either way.)
        const int n_stride = ((B + 63) / 64) * 64;
        if (static_cast<size_t>(4) * n_stride * max_rank <= part_floats)
            return launch_lora_pair_mma(t1, t2, xs, ys, acts, n_br, B, D, max_rank, part, n_stride, s);
    }
    // large batches: a CTA accumulates 8 sub-chunks of 64 rows, so that the up projection adds
    // 8x fewer partial sums per right-hand side; the groups of 8 right-hand sides are grid.z
    const int rep = lora_rep(B);
    const int chunks = (n_chunks + rep - 1) / rep, groups = (B + kLmMaxN - 1) / kLmMaxN;
    d.part = part; d.ldx = D; d.n_chunks = chunks; d.max_rank = max_rank; d.rep = rep;
    u.part = part; u.ldy = D; u.n_chunks = chunks; u.max_rank = max_rank;
    d.n_stride = u.n_stride = groups * kLmMaxN;
    d.n_cols = u.n_cols = B;
    for (int i = 0; i < n_br; ++i) { d.x[i] = xs[i]; u.y[i] = ys[i]; }
    if (rep > 1) launch_pdl(lora_down_kernel<true>, dim3(chunks, n_br, groups), dim3(256), 0, s, d);
    else launch_pdl(lora_down_kernel<false>, dim3(chunks, n_br, groups), dim3(256), 0, s, d);
    launch_pdl(lora_up_kernel, dim3((max_cols + kLuCols - 1) / kLuCols, n_br, groups), dim3(256), 0, s, u);
    return RWKVQ_OK;
}

}  // namespace

extern "C" {

void rwkvq_profiling_tcb_exact(int on) { g_tcb_exact = on < 0 ? -2 : (on ? 1 : 0); }      // rwkvq_profiling.h

int rwkvq_seq_embed_ln0(const rwkvq_qtensor* emb, const int64_t* tokens, const float* ln_w, const float* ln_b, float* x,
                        int64_t n_tokens, int D, void* stream) {
    int rc = validate_qtensor(emb, "rwkvq_seq_embed_ln0");
    if (rc) return rc;
    RWKVQ_REQUIRE(tokens && ln_w && ln_b && x, RWKVQ_E_NULL, "rwkvq_seq_embed_ln0: null pointer");
    RWKVQ_REQUIRE(n_tokens >= 1 && emb->cols == D && D <= kRowThreads * kRowPer, RWKVQ_E_SHAPE,
                  "rwkvq_seq_embed_ln0: %lld tokens, table [%d, %d], D %d (at most %d)", (long long)n_tokens, emb->rows, emb->cols, D,
                  kRowThreads * kRowPer);
    launch_pdl(embed_ln0_kernel, dim3(static_cast<unsigned>(n_tokens)), dim3(kRowThreads), 0, static_cast<cudaStream_t>(stream),
               make_view(*emb), reinterpret_cast<const long long*>(tokens), ln_w, ln_b, x, D);
    return check_launch("rwkvq_seq_embed_ln0");
}

int rwkvq_seq_layer_norm(const float* x, const float* ln_w, const float* ln_b, float* out, int64_t n_rows, int D, void* stream) {
    RWKVQ_REQUIRE(x && ln_w && ln_b && out, RWKVQ_E_NULL, "rwkvq_seq_layer_norm: null pointer");
    RWKVQ_REQUIRE(n_rows >= 1 && D >= 1 && D <= kRowThreads * kRowPer, RWKVQ_E_SHAPE, "rwkvq_seq_layer_norm: %lld rows of %d (at most %d)",
                  (long long)n_rows, D, kRowThreads * kRowPer);
    launch_pdl(D <= 8 * kRowThreads ? ln_shift_mix_kernel<0, 8> : ln_shift_mix_kernel<0, kRowPer>, dim3(static_cast<unsigned>(n_rows)), dim3(kRowThreads), 0, static_cast<cudaStream_t>(stream), x,
               ln_w, ln_b, static_cast<float*>(nullptr), static_cast<const float*>(nullptr), out, static_cast<int>(n_rows), D,
               static_cast<__half*>(nullptr), static_cast<__half*>(nullptr), static_cast<__half*>(nullptr), static_cast<float*>(nullptr), 0,
               static_cast<float*>(nullptr), static_cast<float*>(nullptr));
    return check_launch("rwkvq_seq_layer_norm");
}

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

    launch_pdl(embed_ln0_kernel, dim3(B), dim3(kRowThreads), 0, s, make_view(m->emb),
               reinterpret_cast<const long long*>(tokens), m->ln0_w, m->ln0_b, w.x, D);
    for (int l = 0; l < m->n_layer; ++l) {
        const rwkvq_layer& L = m->layers[l];
        const bool layer0 = l == 0;
        // ---- time mix
        // the row maxima feed the small-batch linears: slots 0-5 the six mix rows, 6 og, 7 xk, 8 hffn, 9 xo
        const bool bp = batch_path(B);
        const bool h16 = bp && batch_fast();          // fp16 rows for the single-term kernels; else fp32 rows and their maxima
        const int ml = mma_layout_of(L.Wr);
        const bool rkv_fused = ml >= 0 && mma_layout_of(L.Wk) == ml && mma_layout_of(L.Wv) == ml && L.Wk.rows == L.Wr.rows &&
                               L.Wv.rows == L.Wr.rows && L.Wk.cols == L.Wr.cols && L.Wv.cols == L.Wr.cols;
        // two-term tcgen05 linears: fp16 pairs of their input rows from the LayerNorm kernels
        const int tcx = tcx_mask(B);
        const bool x_rkv = (tcx & 1) && rkv_fused && gemm_tcb_ok(L.Wr) && gemm_tcb_ok(L.Wk) && gemm_tcb_ok(L.Wv);
        const bool x_key = (tcx & 2) && mma_layout_of(L.Wfk) >= 0 && gemm_tcb_ok(L.Wfk);
        float* am = bp ? w.amax : nullptr;
        float *am_og = bp ? w.amax + 6 * B : nullptr, *am_xk = bp ? w.amax + 7 * B : nullptr;
        float *am_h = bp ? w.amax + 8 * B : nullptr;
        launch_pdl(D <= 8 * kRowThreads ? ln_shift_mix_kernel<6, 8> : ln_shift_mix_kernel<6, kRowPer>, dim3(B), dim3(kRowThreads), 0, s, w.x, L.ln1_w, L.ln1_b, tshift[l], L.x_mix, w.xs, B, D,
                   (h16 || x_rkv) ? w.xs16 : static_cast<__half*>(nullptr), x_rkv ? w.xs16lo : static_cast<__half*>(nullptr),
                   x_rkv ? w.xs_sum : static_cast<__half*>(nullptr), am, 0b001101, am_og, am_h);      // scales of the r, k, v rows
        float *xr = w.xs, *xw = w.xs + BD, *xk = w.xs + 2 * BD, *xv = w.xs + 3 * BD, *xa = w.xs + 4 * BD,
              *xg = w.xs + 5 * BD;
        float *r = w.rkv, *k = w.rkv + BD, *v = w.rkv + 2 * BD;
        SideLane* lane = side_lane(s);
        cudaStream_t s_lora = s;
        if (lane) {                                  // fork: the LoRA branches leave the chain here
            if (cudaEventRecord(lane->fork, s) != cudaSuccess || cudaStreamWaitEvent(lane->stream, lane->fork, 0) != cudaSuccess)
                return fail(RWKVQ_E_LAUNCH, "rwkvq_decode_step: fork onto the side stream failed");
            s_lora = lane->stream;
        }
        // Up to 16 streams the LoRA pair (two dependent launches) is the longer of the two branches: it then
        // stays on the caller's stream, where its first kernel starts programmatically behind the LayerNorm
        // and stages its weights while that still runs, and r / k / v take the side stream.
        cudaStream_t s_rkv = s;
        if (lane && B <= 16) { s_rkv = lane->stream; s_lora = s; }
        if (B == 1 && ml >= 0 && mma_layout_of(L.Wk) == ml && mma_layout_of(L.Wv) == ml && L.Wk.rows == D &&
            L.Wv.rows == D && L.Wr.rows == D && L.Wk.cols == D && L.Wv.cols == D && L.Wr.cols == D) {
            // r, k, v in one launch: three matrices, three inputs (rows 0, 2, 3 of xs)
            for (const rwkvq_qtensor* t : {&L.Wr, &L.Wk, &L.Wv}) {
                rc = validate_qtensor(t, "rwkvq_decode_step(r/k/v)");
                if (rc) return rc;
            }
            const rwkvq_qtensor three[3] = {L.Wr, L.Wk, L.Wv};
            const void* x_each[3] = {xr, xk, xv};
            rc = launch_gemv_mma(ml, three, 3, xr, RWKVQ_F32, D, r, D, RWKVQ_EPI_NONE, nullptr, 1, s_rkv, x_each, w.gscratch);
            if (rc) return rc;
        } else if (bp && rkv_fused) {
            for (const rwkvq_qtensor* t : {&L.Wr, &L.Wk, &L.Wv}) {
                rc = validate_qtensor(t, "rwkvq_decode_step(r/k/v)");
                if (rc) return rc;
            }
            const rwkvq_qtensor three[3] = {L.Wr, L.Wk, L.Wv};
            const void* x3[3] = {w.xs16, w.xs16 + 2 * BD, w.xs16 + 3 * BD};
            const void* x3lo[3] = {w.xs16lo, w.xs16lo + 2 * BD, w.xs16lo + 3 * BD};
            const size_t BS = static_cast<size_t>(B) * (D / 128) * 8;     // block sums of one mix row
            const void* x3sum[3] = {w.xs_sum, w.xs_sum + 2 * BS, w.xs_sum + 3 * BS};
            if (!h16 && !x_rkv) { x3[0] = xr; x3[1] = xk; x3[2] = xv; }
            const float* a3[3] = {am, am + 2 * B, am + 3 * B};
            float* y3[3] = {r, k, v};
            if (x_rkv)
                rc = launch_gemm_tcb(three, 3, x3, true, a3, B, D, y3, D, RWKVQ_EPI_NONE, nullptr, nullptr, w.status, s_rkv, true, x3lo, x3sum);
            else if (tcb_pays(B) && gemm_tcb_ok(L.Wr))
                rc = launch_gemm_tcb(three, 3, x3, h16, a3, B, D, y3, D, RWKVQ_EPI_NONE, nullptr, nullptr, w.status, s_rkv);
            else
                rc = launch_gemv_batch(three, 3, x3, h16, a3, B, D, y3, D, RWKVQ_EPI_NONE, nullptr, nullptr, s_rkv);
            if (rc) return rc;
        } else {
            rc = linear(&L.Wr, xr, B, D, r, D, RWKVQ_EPI_NONE, nullptr, w.gscratch, w.gemm_ws, s_rkv, h16 ? w.xs16 : nullptr, am, nullptr, w.status);
            if (rc) return rc;
            rc = linear(&L.Wk, xk, B, D, k, D, RWKVQ_EPI_NONE, nullptr, w.gscratch, w.gemm_ws, s_rkv,
                        h16 ? w.xs16 + 2 * BD : nullptr, bp ? am + 2 * B : nullptr, nullptr, w.status);
            if (rc) return rc;
            rc = linear(&L.Wv, xv, B, D, v, D, RWKVQ_EPI_NONE, nullptr, w.gscratch, w.gemm_ws, s_rkv,
                        h16 ? w.xs16 + 3 * BD : nullptr, bp ? am + 3 * B : nullptr, nullptr, w.status);
            if (rc) return rc;
        }
        float *yw = w.yl, *ya = w.yl + BD, *yv = w.yl + 2 * BD, *yg = w.yl + 3 * BD;
        {
            const rwkvq_qtensor* t1[4] = {&L.w1, &L.a1, &L.g1, &L.v1};
            const rwkvq_qtensor* t2[4] = {&L.w2, &L.a2, &L.g2, &L.v2};
            const float* x1[4] = {xw, xa, xg, xv};
            float* y2[4] = {yw, ya, yg, yv};
            const int act[4] = {1, 0, 2, 0};       // tanh (decay), none, sigmoid (gate), none
            rc = lora_pair(t1, t2, x1, y2, act, layer0 ? 3 : 4, B, D, m->max_rank, w.part, w.part_floats, w.n_chunks, s_lora);
            if (rc) return rc;
        }
        if (lane) {                                  // join before the time-mix core
            if (cudaEventRecord(lane->join, lane->stream) != cudaSuccess || cudaStreamWaitEvent(s, lane->join, 0) != cudaSuccess)
                return fail(RWKVQ_E_LAUNCH, "rwkvq_decode_step: join of the side stream failed");
        }
        TmixCoreArgs tc{r, k, v, yw, ya, layer0 ? nullptr : yv, yg, L.w0, L.a0, L.v0, L.k_k, L.k_a, L.r_k,
                        L.lnx_w, L.lnx_b, w.v_first, wkv[l], w.og, D, H, layer0 ? 1 : 0, am_og};
        launch_pdl(tmix_core_kernel, dim3(H, B), dim3(256), 0, s, tc);
        rc = linear(&L.Wo, w.og, B, D, w.x, D, RWKVQ_EPI_ADD, w.x, w.gscratch, w.gemm_ws, stream, nullptr, am_og, nullptr, w.status);
        if (rc) return rc;
        // ---- channel mix
        launch_pdl(D <= 8 * kRowThreads ? ln_shift_mix_kernel<1, 8> : ln_shift_mix_kernel<1, kRowPer>, dim3(B), dim3(kRowThreads), 0, s, w.x, L.ln2_w, L.ln2_b, cshift[l], L.ffn_x_k, w.xk, B, D,
                   (h16 || x_key) ? w.xk16 : static_cast<__half*>(nullptr), x_key ? w.xk16lo : static_cast<__half*>(nullptr),
                   x_key ? w.xk_sum : static_cast<__half*>(nullptr), am_xk, 1, static_cast<float*>(nullptr), static_cast<float*>(nullptr));
        rc = linear(&L.Wfk, w.xk, B, D, w.hffn, F, RWKVQ_EPI_RELU2, nullptr, w.gscratch, w.gemm_ws, stream, (h16 || x_key) ? w.xk16 : nullptr,
                    am_xk, am_h, w.status, x_key ? w.xk16lo : nullptr, x_key ? w.xk_sum : nullptr);
        if (rc) return rc;
        rc = linear(&L.Wfv, w.hffn, B, F, w.x, D, RWKVQ_EPI_ADD, w.x, w.gscratch, w.gemm_ws, stream, nullptr, am_h, nullptr, w.status);
        if (rc) return rc;
    }
    float* am_xo = batch_path(B) ? w.amax + 9 * B : nullptr;
    const bool x_head = (tcx_mask(B) & 4) && mma_layout_of(m->head) >= 0 && gemm_tcb_ok(m->head);
    const bool xo_h16 = (am_xo && batch_fast()) || x_head;
    launch_pdl(D <= 8 * kRowThreads ? ln_shift_mix_kernel<0, 8> : ln_shift_mix_kernel<0, kRowPer>, dim3(B), dim3(kRowThreads), 0, s, w.x, m->lnout_w, m->lnout_b, static_cast<float*>(nullptr), static_cast<const float*>(nullptr), w.xo, B, D,
               xo_h16 ? w.xo16 : static_cast<__half*>(nullptr), x_head ? w.xo16lo : static_cast<__half*>(nullptr),
               x_head ? w.xo_sum : static_cast<__half*>(nullptr), am_xo, 1, static_cast<float*>(nullptr), static_cast<float*>(nullptr));
    rc = linear(&m->head, w.xo, B, D, lg, V, RWKVQ_EPI_NONE, nullptr, w.gscratch, w.gemm_ws, stream, xo_h16 ? w.xo16 : nullptr, am_xo, nullptr,
                w.status, x_head ? w.xo16lo : nullptr, x_head ? w.xo_sum : nullptr);
    if (rc) return rc;
    if (next_tokens) {
        float* pv = w.argv;
        int* pi = reinterpret_cast<int*>(w.argv + static_cast<size_t>(B) * kArgSlices);
        launch_pdl(argmax_partial_kernel, dim3(kArgSlices, B), dim3(256), 0, s, static_cast<const float*>(lg), pv, pi, V);
        launch_pdl(argmax_final_kernel, dim3(B), dim3(kArgSlices), 0, s, static_cast<const float*>(pv), static_cast<const int*>(pi), reinterpret_cast<long long*>(next_tokens), V);
    }
    return check_launch("rwkvq_decode_step");
}

}  // extern "C"
