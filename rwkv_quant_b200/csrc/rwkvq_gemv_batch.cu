// Quantized linear for a small batch of right-hand sides (3..64 decode streams, short verify
// runs): every packed weight byte is read ONCE for the whole batch.
//
//     y[n, o] = epi( sum_c W[o, c] x[n, c] ),   n < N
//
// Where the single-vector kernel (rwkvq_gemv_mma.cuh) spends its MMA columns on digits of one
// activation vector, this kernel puts the tokens there: mma.sync.m16n8k16 (f16 x f16 -> f32)
// with the weights as the 16-row operand and 8 tokens per MMA.
//   * a CTA of 8 warps works on groups of 128 or 256 output rows (a warp owns a 16-row tile, two
//     in turn for 256); thread (g, t) streams the codes of rows g, g+8 for blocks 2t, 2t+1 of each
//     group of 8 blocks with the same 128-bit loads from the file layout as the single-vector
//     kernel (load_frag), one group ("iteration") ahead;
//   * the codes become fp16 weights in registers: bytes -> halves by a byte permute onto the
//     exponent pattern of 1024 and one subtract; then, in the default two-term form (EX below),
//     the product with the block scale and its exact rounding error, or, in the single-term form,
//     fp16(q*s + m) by one fused multiply-add per two weights (rounded once: the operand
//     precision of the prefill GEMM).  Block scale and min ARE fp16 values by the codec's definition;
//   * which four k an MMA slot of a thread holds is free as long as both operands agree, so a
//     thread feeds its OWN block's weights (the block whose scale it decoded) and the
//     activations are staged in shared memory in exactly that order: per MMA step the 8 tokens
//     x 4 quad lanes x 4 halves of a warp form 256 contiguous bytes;
//   * activations arrive either as fp16 rows already scaled per token by a power of two (what the
//     LayerNorm kernels of the decode step write: half the bytes, a plain permuting copy) or as
//     fp32 with max|x| of every token known (written by their producer, or by a one-block-per-
//     token pre-pass for the stand-alone entry point): scaled and rounded to fp16 in ONE pass with
//     all loads in flight.  A CTA stages its whole K slice once when that fits (else per chunk);
//     the scale is undone on the fp32 accumulators.  What bounds this phase is the L2 -> SM
//     traffic of the activation rows, re-read by every row group: hence fp16 rows and 256-row
//     groups where the grid allows;
//   * the K loop is split over a thread-block CLUSTER (up to 8 CTAs); the clusters of a launch
//     walk the row groups persistently.  Per row group each CTA leaves its partial tile in its
//     shared memory and, after one cluster barrier, every CTA adds a slice of the tile over all
//     ranks through distributed shared memory in rank order (deterministic, no global scratch,
//     no atomics on the data), applies the epilogue and stores.
// No wait in this kernel spins: the only synchronisation is the hardware cluster barrier.
#include <cooperative_groups.h>

#include <algorithm>
#include <cstdlib>

#include "rwkvq_gemv_mma.cuh"

namespace cg = cooperative_groups;

namespace rwkvq {

constexpr int kBtWarps = 8;
constexpr int kBtThreads = kBtWarps * 32;
constexpr int kBtStepPad = 16;           // bytes between MMA steps in shared memory (bank spread of the staging stores)
constexpr int kBtMaxSmem = 110 * 1024;   // two CTAs per SM

struct BatchArgs {
    QView t[kMmaMaxFused];
    const float* x[kMmaMaxFused];        // [N, ldx] fp32 per matrix, or null when x16 is given
    const float* amax[kMmaMaxFused];     // with x:   [N] max|x| of every token (inf / nan when the row is not finite)
    const __half* x16[kMmaMaxFused];     // [N, ldx] fp16 rows = x * 2^s per token
    const float* unscale[kMmaMaxFused];  // with x16: [N] 2^-s
    float* y[kMmaMaxFused];              // [N, ldy]
    const float* resid[kMmaMaxFused];    // [N, ldy] or null
    float* amax_out[kMmaMaxFused];       // optional [N]: max|y| per token is merged into it (atomic max; the caller zeroes it)
    long long ldx, ldy;
    int n_tokens;
    int epilogue;
    int tiles_per_cta;                   // 16-row tiles of one row group (8 or 16)
    int its_per_cta;                     // iterations (Geo::KI columns each) of one CTA's K slice
    int chunk_its;                       // iterations staged per shared-memory chunk
    int ks;                              // CTAs along K = cluster size
    unsigned long long* trace;           // profiling aid (rwkvq_profiling.h): 8 global-timer marks of CTA (0,0,0), or null
};

__device__ __forceinline__ void bt_mark(const BatchArgs& a, int slot) {
    if (a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        a.trace[slot] = t;
    }
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// sb6: (s, m) of blocks 2t, 2t+1 as half2 pairs; the arithmetic of sb6_pair_scales without the
// widening to fp32.  The codec's floor max(s, 1e-8) is below the fp16 range and is dropped: a
// block whose scale code or super-scale is zero dequantises to its min alone (|dw| <= 63e-8).
__device__ __forceinline__ void sb6_pair_scales_h2(const uint4& rec, int t, __half2& hs, __half2& hm) {
    const uint32_t w = (t & 2) ? ((t & 1) ? rec.w : rec.z) : ((t & 1) ? rec.y : rec.x);
    const uint32_t dd = __byte_perm(rec.x, rec.y, 0x7373);
    const uint32_t dmm = __byte_perm(rec.z, rec.w, 0x7373);
    const uint32_t qs = (w & 0x3Fu) | ((w << 10) & 0x003F0000u) | 0x64006400u;
    const uint32_t qm = ((w >> 12) & 0x3Fu) | ((w >> 2) & 0x003F0000u) | 0x64006400u;
    hs = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&qs), __float2half2_rn(1024.f)),
                 *reinterpret_cast<const __half2*>(&dd));
    hm = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&qm), __float2half2_rn(1055.f)),
                 *reinterpret_cast<const __half2*>(&dmm));
}
__device__ __forceinline__ __half2 sym_pair_scales_h2(uint32_t q_lo, uint32_t q_hi, uint32_t d_bits, int t) {
    const uint32_t w = (t & 2) ? q_hi : q_lo;
    const uint32_t two = (t & 1) ? (w >> 16) : (w & 0xFFFFu);
    const uint32_t u = ((two ^ 0x8080u) & 0xFFu) | (((two ^ 0x8080u) << 8) & 0x00FF0000u) | 0x64006400u;
    const uint32_t dd = d_bits | (d_bits << 16);
    return __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&u), __float2half2_rn(1152.f)),
                   *reinterpret_cast<const __half2*>(&dd));
}

// Four byte codes -> two half2 of weights.  `bias`: what the byte pattern 0x6400 | code exceeds
// the signed code by (1024 for unsigned codes, 1056 for codes stored +32, 1152 for int8 ^ 0x80).
template <bool HAS_MIN>
__device__ __forceinline__ void cvt4(uint32_t w, __half2 bias, __half2 s2, __half2 m2, uint32_t& lo, uint32_t& hi) {
    const uint32_t p01 = __byte_perm(w, 0x64646464u, 0x4140), p23 = __byte_perm(w, 0x64646464u, 0x4342);
    const __half2 q01 = __hsub2(*reinterpret_cast<const __half2*>(&p01), bias);
    const __half2 q23 = __hsub2(*reinterpret_cast<const __half2*>(&p23), bias);
    const __half2 w01 = HAS_MIN ? __hfma2(q01, s2, m2) : __hmul2(q01, s2);
    const __half2 w23 = HAS_MIN ? __hfma2(q23, s2, m2) : __hmul2(q23, s2);
    lo = *reinterpret_cast<const uint32_t*>(&w01);
    hi = *reinterpret_cast<const uint32_t*>(&w23);
}

// Four codes times their block scale as TWO fp16 terms per weight: p = fp16(q*s) and the rounding
// error of that product, which a fused multiply-add recovers exactly (q*s has at most 19
// significant bits, p keeps the top 11).  p + e = q*s up to the fp16 subnormal quantum (6e-8
// absolute).  The block min is not folded in: it multiplies the block's activation sum instead.
__device__ __forceinline__ void cvt4x(uint32_t w, __half2 bias, __half2 s2, uint32_t& p01, uint32_t& p23, uint32_t& e01,
                                      uint32_t& e23) {
    const uint32_t b01 = __byte_perm(w, 0x64646464u, 0x4140), b23 = __byte_perm(w, 0x64646464u, 0x4342);
    const __half2 q01 = __hsub2(*reinterpret_cast<const __half2*>(&b01), bias);
    const __half2 q23 = __hsub2(*reinterpret_cast<const __half2*>(&b23), bias);
    const __half2 w01 = __hmul2(q01, s2), w23 = __hmul2(q23, s2);
    const __half2 r01 = __hfma2(q01, s2, __hneg2(w01)), r23 = __hfma2(q23, s2, __hneg2(w23));
    p01 = *reinterpret_cast<const uint32_t*>(&w01);
    p23 = *reinterpret_cast<const uint32_t*>(&w23);
    e01 = *reinterpret_cast<const uint32_t*>(&r01);
    e23 = *reinterpret_cast<const uint32_t*>(&r23);
}

// Shared-memory order of the staged activations.  An iteration covers KI columns = 8 blocks;
// thread t of a quad owns blocks 2t + h.  MMA step s = ((h * NJ) + j) * 2 + half takes, from
// every quad lane, the 4 weights at offset koff(j, half) of its block, so element
// (token n, lane t, e < 4) of step s is x[n][it * KI + (2t + h) * BLK + koff + e].
template <int L> struct BtGeo {
    static constexpr int NJ = (L <= ML_SB6_6) ? 4 : 2;
    static constexpr int STEPS = Geo<L>::KI / 16;
    __device__ static constexpr int koff(int j, int half) { return (L <= ML_SB6_6) ? half * 16 + 4 * j : j * 8 + half * 4; }
};



// EX: both operands as two fp16 terms (x: hi + lo of the scaled fp32 value; W: q*s as product and
// rounding error, cvt4x) and three MMAs per step (hi*hi + lo*hi + hi*lo); the block mins, fp16
// values by the codec's definition, multiply the per-block sums of the activations in one more
// pair of MMAs per iteration (k = the 8 blocks, which a thread holds in exactly the fragment order
// it decoded them).  That leaves the fp32 accumulation as the only rounding: the result agrees
// with an fp32 dequantise-and-multiply to ~1e-6 instead of ~5e-4.  The activations are fp32 rows
// with their max, scaled to at most 2^9 so that a block sum stays inside the fp16 range; the hi and
// lo halves of a lane's four activations sit side by side (one 128-bit load per MMA triple).
template <int L, int NT, bool EX>      // NT: 8-token tiles of the MMA N dimension
__global__ void __launch_bounds__(kBtThreads, 2) gemv_batch_kernel(const BatchArgs a) {
    using G = Geo<L>;
    using BG = BtGeo<L>;
    constexpr int N8 = NT * 8;
    constexpr int SP = N8 * 32 * (EX ? 2 : 1) + kBtStepPad;          // bytes per MMA step
    constexpr bool SB6 = L <= ML_SB6_6;
    constexpr int SUMB = (EX && SB6) ? N8 * 32 : 0;   // per iteration: the 8 block sums of every token, 8 hi then 8 lo halves
    constexpr int ITB = BG::STEPS * SP + SUMB;        // bytes per staged iteration
    extern __shared__ __align__(16) unsigned char smem[];
    cg::cluster_group cluster = cg::this_cluster();

    const QView& q = a.t[blockIdx.y];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int ks = a.ks, rank = static_cast<int>(blockIdx.x) % ks;
    const int cid = static_cast<int>(blockIdx.x) / ks, n_clusters = static_cast<int>(gridDim.x) / ks;
    const int n0 = blockIdx.z * N8;                                     // first token of this CTA's group
    const int nn = min(N8, a.n_tokens - n0);
    const int tpc = a.tiles_per_cta, R = tpc * 16, RP = R + 4;
    const int n_tiles = (q.rows + 15) >> 4;
    const int n_rg = (n_tiles + tpc - 1) / tpc;
    const int it_base = rank * a.its_per_cta;
    const int n_chunks = (a.its_per_cta + a.chunk_its - 1) / a.chunk_its;
    const int my_tiles = tpc / kBtWarps;                                // 1 or 2 (1 whenever the K slice is chunked)

    float* sc = reinterpret_cast<float*>(smem);                         // [N8] scale, [N8] its inverse
    float* un = sc + N8;
    float* omax = un + N8;                                              // [N8] max|y| of this CTA's stores (as int bits)
    float* part = omax + N8;                                            // [N8][RP] partial sums
    unsigned char* xs = reinterpret_cast<unsigned char*>(part + N8 * RP);   // staged fp16 activations

    // flat item sequence (row group, tile, iteration) of this warp, for the prefetch
    const int my_rg = cid < n_rg ? (n_rg - cid + n_clusters - 1) / n_clusters : 0;
    const int n_items = my_rg * my_tiles * a.its_per_cta;
    int i_n = 0, i_rg = cid, i_ti = 0, i_it = 0;
    Frag<L> nxt;
    auto fetch_next = [&]() {
        const int tile = i_rg * tpc + warp + i_ti * kBtWarps;
        if (i_n < n_items && tile < n_tiles) {
            const int r0 = min(tile * 16 + g, q.rows - 1), r1 = min(tile * 16 + g + 8, q.rows - 1);
            load_frag<L>(nxt, q, r0, r1, it_base + i_it, t);
        }
        ++i_n;
        if (++i_it == a.its_per_cta) {
            i_it = 0;
            if (++i_ti == my_tiles) { i_ti = 0; i_rg += n_clusters; }
        }
    };
    bt_mark(a, 0);
    pdl_launch_dependents();
    fetch_next();                          // weights do not depend on the producer of x
    pdl_wait();
    bt_mark(a, 1);

    const bool is16 = a.x16[blockIdx.y] != nullptr;
    if (threadIdx.x < N8) {
        const int n = threadIdx.x;
        float s1 = 1.f, u1 = 1.f;
        if (is16) {
            if (n < nn) u1 = __ldcg(a.unscale[blockIdx.y] + n0 + n);
        } else {
            // |x| * 2^(14 - e) <= 2^14 with amax <= 2^e; a non-finite row keeps scale 1 and propagates
            const float am = n < nn ? __ldcg(a.amax[blockIdx.y] + n0 + n) : 0.f;
            if (am > 0.f && am < INFINITY) {
                int e = 0;
                frexpf(am, &e);
                e = max(-100, e);                       // 2^(14 - e) must stay finite
                s1 = ldexpf(1.f, (EX ? 9 : 14) - e);
                u1 = ldexpf(1.f, e - (EX ? 9 : 14));
            }
        }
        sc[n] = s1;
        un[n] = u1;
        omax[n] = 0.f;
    }
    __syncthreads();

    // shared-memory slot of the 4 activations at column k (multiple of 4) of the staged chunk, token n
    auto slot_of = [&](int k, int n) -> unsigned char* {
        const int it_l = k / G::KI, rem = k % G::KI;
        const int blk = rem / G::BLK, off = rem % G::BLK;
        const int tt = blk >> 1, h = blk & 1;
        const int half = SB6 ? (off >> 4) : ((off >> 2) & 1), j = SB6 ? ((off >> 2) & 3) : (off >> 3);
        const int step = ((h * BG::NJ) + j) * 2 + half;
        return xs + static_cast<size_t>(it_l) * ITB + step * SP + (n * 32 + tt * 8) * (EX ? 2 : 1);
    };
    // stage columns [kbase, kbase + cits * KI) of every token: one pass, 8 vector loads in flight per thread
    auto stage = [&](int ch) {
        const int cits = min(a.chunk_its, a.its_per_cta - ch * a.chunk_its);
        const int kbase = (it_base + ch * a.chunk_its) * G::KI;
        if (is16) {
            const __half* xg = a.x16[blockIdx.y] + static_cast<size_t>(n0) * a.ldx + kbase;
            const int v_row = cits * G::KI / 8;                  // 16-byte vectors (8 halves) per token
            const int total = N8 * v_row;
            for (int base = threadIdx.x; base < total; base += 8 * kBtThreads) {
                uint4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int idx = base + u * kBtThreads;
                    const int n = idx / v_row, k8 = idx - n * v_row;
                    v[u] = (idx < total && n < nn) ? __ldcg(reinterpret_cast<const uint4*>(xg + static_cast<size_t>(n) * a.ldx) + k8)
                                                   : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int idx = base + u * kBtThreads;
                    if (idx >= total) break;
                    const int n = idx / v_row, k8 = idx - n * v_row;
                    *reinterpret_cast<uint2*>(slot_of(8 * k8, n)) = make_uint2(v[u].x, v[u].y);
                    *reinterpret_cast<uint2*>(slot_of(8 * k8 + 4, n)) = make_uint2(v[u].z, v[u].w);
                }
            }
        } else {
            const float* xg = a.x[blockIdx.y] + static_cast<size_t>(n0) * a.ldx + kbase;
            const int v_row = cits * G::KI / 4;                  // float4 per token
            const int total = N8 * v_row;
            for (int base = threadIdx.x; base < total; base += 8 * kBtThreads) {
                float4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int idx = base + u * kBtThreads;
                    const int n = idx / v_row, k4 = idx - n * v_row;
                    v[u] = (idx < total && n < nn) ? __ldcg(reinterpret_cast<const float4*>(xg + static_cast<size_t>(n) * a.ldx) + k4)
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int idx = base + u * kBtThreads;
                    if (idx >= total) break;
                    const int n = idx / v_row, k4 = idx - n * v_row;
                    const float s1 = sc[n];
                    const __half2 h01 = __floats2half2_rn(v[u].x * s1, v[u].y * s1);
                    const __half2 h23 = __floats2half2_rn(v[u].z * s1, v[u].w * s1);
                    uint2 pk;
                    pk.x = *reinterpret_cast<const uint32_t*>(&h01);
                    pk.y = *reinterpret_cast<const uint32_t*>(&h23);
                    unsigned char* slot = slot_of(4 * k4, n);
                    if (!EX) *reinterpret_cast<uint2*>(slot) = pk;
                    if (EX) {
                        const float2 b01 = __half22float2(h01), b23 = __half22float2(h23);
                        const __half2 l01 = __floats2half2_rn(v[u].x * s1 - b01.x, v[u].y * s1 - b01.y);
                        const __half2 l23 = __floats2half2_rn(v[u].z * s1 - b23.x, v[u].w * s1 - b23.y);
                        *reinterpret_cast<uint4*>(slot) = make_uint4(pk.x, pk.y, *reinterpret_cast<const uint32_t*>(&l01),
                                                                     *reinterpret_cast<const uint32_t*>(&l23));
                        if (SB6) {      // 8 consecutive lanes hold the 32 columns of one block (every pass of the CTA is full)
                            float bs = (v[u].x * s1 + v[u].y * s1) + (v[u].z * s1 + v[u].w * s1);
                            bs += __shfl_xor_sync(0xFFFFFFFFu, bs, 1);
                            bs += __shfl_xor_sync(0xFFFFFFFFu, bs, 2);
                            bs += __shfl_xor_sync(0xFFFFFFFFu, bs, 4);
                            if ((k4 & 7) == 0) {
                                const int kk = 4 * k4, it_l = kk / G::KI, blk = (kk % G::KI) / G::BLK;
                                __half* sums = reinterpret_cast<__half*>(xs + static_cast<size_t>(it_l) * ITB + BG::STEPS * SP + n * 32);
                                const __half sh = __float2half_rn(bs);
                                sums[blk] = sh;
                                sums[8 + blk] = __float2half_rn(bs - __half2float(sh));
                            }
                        }
                    }
                }
            }
        }
    };
    if (n_chunks == 1) {
        stage(0);
        __syncthreads();
    }
    bt_mark(a, 2);
    const __half2 bias = __float2half2_rn(L == ML_SYM6 ? 1056.f : (L == ML_SYM8 || L == ML_RTN8) ? 1152.f : 1024.f);
    float* y = a.y[blockIdx.y] + static_cast<size_t>(n0) * a.ldy;
    const float* resid = a.resid[blockIdx.y] ? a.resid[blockIdx.y] + static_cast<size_t>(n0) * a.ldy : nullptr;
    const bool vec_io = (a.ldy % 4 == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0) &&
                        (resid == nullptr || (reinterpret_cast<uintptr_t>(resid) & 15) == 0);

    // the staged iterations [0, cits) of one tile: c += W x
    auto run_its = [&](int tile, int cits, float (&c)[NT][4]) {
        for (int il = 0; il < cits; ++il) {
            const Frag<L> cur = nxt;
            fetch_next();
            if (tile >= n_tiles) continue;
            const unsigned char* xrow = xs + static_cast<size_t>(il) * ITB + (g * 32 + t * 8) * (EX ? 2 : 1);
            if (EX) {
                __half2 sa, sb, ma = __float2half2_rn(0.f), mb = ma;
                if (SB6) {
                    sb6_pair_scales_h2(cur.ma, t, sa, ma);
                    sb6_pair_scales_h2(cur.mb, t, sb, mb);
                } else if (L == ML_RTN8) {
                    sa = __half2half2(__ushort_as_half(static_cast<unsigned short>(cur.ma.z)));
                    sb = __half2half2(__ushort_as_half(static_cast<unsigned short>(cur.mb.z)));
                } else {
                    sa = sym_pair_scales_h2(cur.ma.x, cur.ma.y, cur.ma.z, t);
                    sb = sym_pair_scales_h2(cur.mb.x, cur.mb.y, cur.mb.z, t);
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const __half2 s0 = h ? __high2half2(sa) : __low2half2(sa), s1 = h ? __high2half2(sb) : __low2half2(sb);
#pragma unroll
                    for (int j = 0; j < BG::NJ; ++j) {
                        uint32_t lo0, hi0, lo1, hi1;
                        a_words<L>(cur.ca, cur.pa, h, j, lo0, hi0);
                        a_words<L>(cur.cb, cur.pb, h, j, lo1, hi1);
                        if (L == ML_SYM8 || L == ML_RTN8) { lo0 ^= 0x80808080u; hi0 ^= 0x80808080u; lo1 ^= 0x80808080u; hi1 ^= 0x80808080u; }
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
                            cvt4x(half ? hi0 : lo0, bias, s0, a0, a2, e0, e2);
                            cvt4x(half ? hi1 : lo1, bias, s1, a1, a3, e1, e3);
                            const unsigned char* xp = xrow + (((h * BG::NJ) + j) * 2 + half) * SP;
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                const uint4 b = *reinterpret_cast<const uint4*>(xp + nt * 512);     // hi (x, y), lo (z, w)
                                mma_f16(c[nt], e0, e1, e2, e3, b.x, b.y);       // small terms first
                                mma_f16(c[nt], a0, a1, a2, a3, b.z, b.w);
                                mma_f16(c[nt], a0, a1, a2, a3, b.x, b.y);
                            }
                        }
                    }
                }
                if (SB6) {      // + m[row][blk] * sum_blk(x): A = the mins of blocks 2t, 2t+1 (k slots 2t, 2t+1), B = the block sums
                    const unsigned char* sp = xs + static_cast<size_t>(il) * ITB + BG::STEPS * SP + g * 32 + t * 4;
                    const uint32_t m0 = *reinterpret_cast<const uint32_t*>(&ma), m1 = *reinterpret_cast<const uint32_t*>(&mb);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const uint32_t bh = *reinterpret_cast<const uint32_t*>(sp + nt * 256);
                        const uint32_t bl = *reinterpret_cast<const uint32_t*>(sp + nt * 256 + 16);
                        mma_f16(c[nt], m0, m1, 0u, 0u, bl, 0u);
                        mma_f16(c[nt], m0, m1, 0u, 0u, bh, 0u);
                    }
                }
                continue;
            }
            __half2 sa, sb, ma = __float2half2_rn(0.f), mb = ma;
            if (SB6) {
                sb6_pair_scales_h2(cur.ma, t, sa, ma);
                sb6_pair_scales_h2(cur.mb, t, sb, mb);
            } else if (L == ML_RTN8) {
                sa = __half2half2(__ushort_as_half(static_cast<unsigned short>(cur.ma.z)));
                sb = __half2half2(__ushort_as_half(static_cast<unsigned short>(cur.mb.z)));
            } else {
                sa = sym_pair_scales_h2(cur.ma.x, cur.ma.y, cur.ma.z, t);
                sb = sym_pair_scales_h2(cur.mb.x, cur.mb.y, cur.mb.z, t);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const __half2 s0 = h ? __high2half2(sa) : __low2half2(sa), s1 = h ? __high2half2(sb) : __low2half2(sb);
                const __half2 m0 = h ? __high2half2(ma) : __low2half2(ma), m1 = h ? __high2half2(mb) : __low2half2(mb);
#pragma unroll
                for (int j = 0; j < BG::NJ; ++j) {
                    uint32_t lo0, hi0, lo1, hi1;
                    a_words<L>(cur.ca, cur.pa, h, j, lo0, hi0);
                    a_words<L>(cur.cb, cur.pb, h, j, lo1, hi1);
                    if (L == ML_SYM8 || L == ML_RTN8) { lo0 ^= 0x80808080u; hi0 ^= 0x80808080u; lo1 ^= 0x80808080u; hi1 ^= 0x80808080u; }
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t a0, a1, a2, a3;
                        cvt4<SB6>(half ? hi0 : lo0, bias, s0, m0, a0, a2);      // row g:     k slots (2t, 2t+1), (2t+8, 2t+9)
                        cvt4<SB6>(half ? hi1 : lo1, bias, s1, m1, a1, a3);      // row g + 8
                        const unsigned char* xp = xrow + (((h * BG::NJ) + j) * 2 + half) * SP;
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const uint2 b = *reinterpret_cast<const uint2*>(xp + nt * 256);
                            mma_f16(c[nt], a0, a1, a2, a3, b.x, b.y);
                        }
                    }
                }
            }
        }
    };
    // undo the token scales and leave the tile for the reduction
    auto put_part = [&](int ti, const float (&c)[NT][4]) {
        const int r = (warp + ti * kBtWarps) * 16 + g;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int n = nt * 8 + 2 * t;
            const float u0 = un[n], u1 = un[n + 1];
            part[n * RP + r] = c[nt][0] * u0;
            part[(n + 1) * RP + r] = c[nt][1] * u1;
            part[n * RP + r + 8] = c[nt][2] * u0;
            part[(n + 1) * RP + r + 8] = c[nt][3] * u1;
        }
    };

    for (int rg = cid; rg < n_rg; rg += n_clusters) {
        if (n_chunks == 1) {
            for (int ti = 0; ti < my_tiles; ++ti) {
                float c[NT][4];
#pragma unroll
                for (int i = 0; i < NT; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
                run_its(rg * tpc + warp + ti * kBtWarps, a.its_per_cta, c);
                put_part(ti, c);
            }
        } else {
            float c[NT][4];
#pragma unroll
            for (int i = 0; i < NT; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
            for (int ch = 0; ch < n_chunks; ++ch) {
                __syncthreads();                   // everyone is done with the chunk staged before
                stage(ch);
                __syncthreads();
                run_its(rg * tpc + warp, min(a.chunk_its, a.its_per_cta - ch * a.chunk_its), c);
            }
            put_part(0, c);
        }
        if (rg == cid) bt_mark(a, 3);
        cluster.sync();
        if (rg == cid) bt_mark(a, 4);
        // ---- add the ks partial tiles in rank order, epilogue, store: float4 groups of 4 rows
        {
            const int g4 = R / 4;
            const int total4 = nn * g4;
            const int per = (total4 + ks - 1) / ks;
            const int lo = rank * per, hi = min(total4, lo + per);
            const int row0 = rg * R;
            for (int i4 = lo + threadIdx.x; i4 < hi; i4 += kBtThreads) {
                const int n = i4 / g4, r = (i4 - n * g4) * 4;
                const int row = row0 + r;
                if (row >= q.rows) continue;
                float4 v[8];
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (k < ks) v[k] = *reinterpret_cast<const float4*>(cluster.map_shared_rank(part, k) + n * RP + r);
                float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (k < ks) { s.x += v[k].x; s.y += v[k].y; s.z += v[k].z; s.w += v[k].w; }
                const size_t o = static_cast<size_t>(n) * a.ldy + row;
                const bool full = vec_io && row + 3 < q.rows;
                if (a.epilogue == RWKVQ_EPI_RELU2) {
                    s.x = fmaxf(s.x, 0.f); s.y = fmaxf(s.y, 0.f); s.z = fmaxf(s.z, 0.f); s.w = fmaxf(s.w, 0.f);
                    s.x *= s.x; s.y *= s.y; s.z *= s.z; s.w *= s.w;
                } else if (a.epilogue == RWKVQ_EPI_ADD) {
                    if (full) {
                        const float4 rv = __ldcg(reinterpret_cast<const float4*>(resid + o));
                        s.x = __fadd_rn(s.x, rv.x); s.y = __fadd_rn(s.y, rv.y); s.z = __fadd_rn(s.z, rv.z); s.w = __fadd_rn(s.w, rv.w);
                    } else {
                        s.x = __fadd_rn(s.x, __ldcg(resid + o));
                        if (row + 1 < q.rows) s.y = __fadd_rn(s.y, __ldcg(resid + o + 1));
                        if (row + 2 < q.rows) s.z = __fadd_rn(s.z, __ldcg(resid + o + 2));
                        if (row + 3 < q.rows) s.w = __fadd_rn(s.w, __ldcg(resid + o + 3));
                    }
                }
                if (full) {
                    *reinterpret_cast<float4*>(y + o) = s;
                } else {
                    y[o] = s.x;
                    if (row + 1 < q.rows) y[o + 1] = s.y;
                    if (row + 2 < q.rows) y[o + 2] = s.z;
                    if (row + 3 < q.rows) y[o + 3] = s.w;
                }
                if (a.amax_out[blockIdx.y] != nullptr) {
                    // |v| as int bits orders like the float; a NaN compares above every number and so survives
                    float m = fabsf(s.x);
                    if (row + 1 < q.rows) m = fmaxf(m, fabsf(s.y)) + 0.f * s.y;
                    if (row + 2 < q.rows) m = fmaxf(m, fabsf(s.z)) + 0.f * s.z;
                    if (row + 3 < q.rows) m = fmaxf(m, fabsf(s.w)) + 0.f * s.w;
                    atomicMax(reinterpret_cast<int*>(omax) + n, __float_as_int(fabsf(m)));
                }
            }
        }
        if (rg == cid) bt_mark(a, 5);
        cluster.sync();          // nobody overwrites or leaves while a peer still reads its partial tile
    }
    if (a.amax_out[blockIdx.y] != nullptr) {
        __syncthreads();
        if (threadIdx.x < nn) {
            const int bits = reinterpret_cast<const int*>(omax)[threadIdx.x];
            if (bits != 0) atomicMax(reinterpret_cast<int*>(a.amax_out[blockIdx.y]) + n0 + threadIdx.x, bits);
        }
    }
    bt_mark(a, 6);
}

// max|x| of every row (one block per row): the pre-pass of the stand-alone entry point; inside
// the decode step the producers of the activations write it themselves.  A non-finite row
// yields inf or nan.
__global__ void __launch_bounds__(256) row_amax_kernel(const float* __restrict__ x, long long ldx, int cols, float* __restrict__ amax,
                                                       int* __restrict__ status) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    if (status != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *status = 0;      // status word of the product kernel that follows
    const float* row = x + static_cast<size_t>(blockIdx.x) * ldx;
    float m = 0.f;
    for (int i = threadIdx.x; i < cols / 4; i += 256) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(row) + i);
        m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        if (!(fabsf(v.x) + fabsf(v.y) + fabsf(v.z) + fabsf(v.w) < INFINITY)) m = INFINITY;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
        amax[blockIdx.x] = m;
    }
}

// RWKVQ_BATCH_FAST=1 in the environment (read once) trades accuracy for speed in the small-batch
// linears: single fp16 operands (relative error ~5e-4 per linear, the arithmetic of the prefill GEMM)
// and, above 32 rows, the tcgen05 kernel.  The default is the two-term kernel.
int g_batch_fast = -1;
bool batch_fast() {
    if (g_batch_fast < 0) {
        const char* e = getenv("RWKVQ_BATCH_FAST");
        g_batch_fast = (e != nullptr && e[0] == '1') ? 1 : 0;
    }
    return g_batch_fast == 1;
}

unsigned long long* g_batch_trace = nullptr;      // set by rwkvq_profiling_batch_trace (rwkvq_profiling.h)
int g_batch_force_ks = 0;                         // profiling aid: cluster size override (0 = the launcher's choice)
int g_batch_force_rows = 0, g_batch_force_cols = 0;   // ... for tensors of this shape only (0: every shape)

namespace {

template <int L, int NT, bool EX>
int launch_bt(BatchArgs& a, int n_mats, int n_groups, int n_clusters, size_t smem, cudaStream_t s) {
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
    if (dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_batch_kernel<L, NT, EX>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBtMaxSmem);
        if (e != cudaSuccess) return fail(RWKVQ_E_LIMIT, "rwkvq_gemv_batch: shared memory attribute: %s", cudaGetErrorString(e));
        if (dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(n_clusters * a.ks, n_mats, n_groups);
    cfg.blockDim = dim3(kBtThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = a.ks; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, gemv_batch_kernel<L, NT, EX>, a);
    if (le != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_gemv_batch: %s", cudaGetErrorString(le));
    return RWKVQ_OK;
}

template <int L>
int launch_bt_l(BatchArgs& a, int n_mats, int rows, int cols, int N, bool exact, cudaStream_t s) {
    using G = Geo<L>;
    const int n_iters = cols / G::KI;
    // The two-term kernel works on 16 tokens at a time (grid.z walks the groups of a larger batch): measured
    // inside the decode graph, two CTAs with 16 tokens each beat one with 32 on every shape (3 MMAs per step
    // make the 32-token tile MMA-issue bound, and its staged K slice no longer fits unchunked), and for
    // K >= 8192 one with 8 beats one with 16.  One exception, measured the same way at 20, 24 and 32 tokens on
    // the ffn-key shapes of the 1.5B and 2.9B models ([8192, 2048], [10240, 2560]): with at most 32 tokens and
    // at least twice as many rows as columns ONE CTA with 32 tokens is 1-5 us faster per launch (the output
    // projection, the ffn value and the head lose with it).
    const bool tall = rows >= 2 * cols && rows <= 16384;
    int nt = exact ? (N <= 8 || (N <= 16 && cols >= 8192) ? 1 : (N > 16 && N <= 32 && tall) ? 4 : 2)
                   : N <= 8 ? 1 : N <= 16 ? 2 : N <= 32 ? 4 : 8;
    const bool forced = g_batch_force_ks > 0 && (g_batch_force_rows == 0 || (g_batch_force_rows == rows && g_batch_force_cols == cols));
    if (forced && (g_batch_force_ks & 64) && nt > 1) nt /= 2;      // profiling: half the token tile, twice the token groups
    if (forced && (g_batch_force_ks & 128) && nt > 1) nt /= 2;     // ... and half again
    const int n8 = nt * 8, n_groups = (N + n8 - 1) / n8;
    const int n_tiles = (rows + 15) / 16;
    const int mats = n_mats * n_groups;
    const size_t step_bytes = static_cast<size_t>(n8) * 32 * (exact ? 2 : 1) + kBtStepPad;
    const size_t it_bytes = step_bytes * (G::KI / 16) + ((exact && L <= ML_SB6_6) ? static_cast<size_t>(n8) * 32 : 0);
    auto fixed_bytes = [&](int tpc) { return static_cast<size_t>(3 * n8) * sizeof(float) + static_cast<size_t>(n8) * (tpc * 16 + 4) * sizeof(float); };
    // Cost model (microseconds of the slowest CTA) over the cluster size ks (a divisor of the iteration
    // count) and the rows per group (128 or 256): activations staged once (L2 -> SM traffic of all
    // row groups together at ~3.5 TB/s), then per row group the products and the cluster reduction.
    const bool half_in = a.x16[0] != nullptr;
    int best_ks = 1, best_tpc = 8;
    double best = 1e30;
    for (int tpc = 8; tpc <= 16; tpc += 8) {
        for (int c = 1; c <= 8; ++c) {
            if (n_iters % c) continue;
            const int ipc = n_iters / c;
            const int max_chunk = static_cast<int>((static_cast<long long>(kBtMaxSmem) - static_cast<long long>(fixed_bytes(tpc))) /
                                                   static_cast<long long>(it_bytes));
            if (max_chunk < 1) continue;
            const bool chunked = ipc > max_chunk;
            if (chunked && tpc != 8) continue;
            const int n_rg = (n_tiles + tpc - 1) / tpc;
            const int slots = std::max(1, (2 * 148) / c);                       // resident clusters (2 CTAs per SM)
            const int clusters = std::max(1, std::min(n_rg, std::max(1, slots / std::max(1, mats))));
            const int rounds = (n_rg + clusters - 1) / clusters;
            const double f = n8 / 64.0;
            const double x_mb = static_cast<double>(clusters) * mats * n8 * cols * (half_in ? 2 : 4) / 1e6 * (chunked ? rounds : 1);
            const double stage_us = 0.8 + x_mb / 3.5;
            const double it_us = (exact ? 1.0 + 3.4 * f : 0.6 + 1.7 * f) * G::KI / 256.0 * (tpc / 8);
            const double red_us = 1.6 + 0.15 * c + 0.5 * f * (tpc / 8);
            const double occupancy = (clusters * c * mats > 148) ? 1.35 : 1.0;  // two CTAs share an SM
            const double t = stage_us + rounds * (ipc * it_us * occupancy + red_us) + (c == 8 ? 0.8 : 0.0);
            if (t < best) { best = t; best_ks = c; best_tpc = tpc; }
        }
    }
    int ks = best_ks, tpc = best_tpc;
    if (forced && (g_batch_force_ks & 15) > 0 && n_iters % (g_batch_force_ks & 15) == 0) {
        ks = g_batch_force_ks & 15;
        if (g_batch_force_ks & 16) tpc = 16;
        if (g_batch_force_ks & 32) tpc = 8;
    }
    a.ks = ks;
    a.its_per_cta = n_iters / ks;
    int max_chunk = static_cast<int>((static_cast<long long>(kBtMaxSmem) - static_cast<long long>(fixed_bytes(tpc))) /
                                     static_cast<long long>(it_bytes));
    if (a.its_per_cta > max_chunk) {
        tpc = 8;
        max_chunk = static_cast<int>((static_cast<long long>(kBtMaxSmem) - static_cast<long long>(fixed_bytes(tpc))) /
                                     static_cast<long long>(it_bytes));
    }
    if (max_chunk < 1) return fail(RWKVQ_E_LIMIT, "rwkvq_gemv_batch: no room for one staged iteration");
    a.chunk_its = std::min(a.its_per_cta, max_chunk);
    a.tiles_per_cta = tpc;
    const int n_rg = (n_tiles + tpc - 1) / tpc;
    const int slots = std::max(1, (2 * 148) / ks);
    const int n_clusters = std::max(1, std::min(n_rg, std::max(1, slots / std::max(1, mats))));
    const size_t smem = fixed_bytes(tpc) + static_cast<size_t>(a.chunk_its) * it_bytes;
    if (exact) {
        switch (nt) {
            case 1: return launch_bt<L, 1, true>(a, n_mats, n_groups, n_clusters, smem, s);
            case 2: return launch_bt<L, 2, true>(a, n_mats, n_groups, n_clusters, smem, s);
            default: return launch_bt<L, 4, true>(a, n_mats, n_groups, n_clusters, smem, s);
        }
    }
    switch (nt) {
        case 1: return launch_bt<L, 1, false>(a, n_mats, n_groups, n_clusters, smem, s);
        case 2: return launch_bt<L, 2, false>(a, n_mats, n_groups, n_clusters, smem, s);
        case 4: return launch_bt<L, 4, false>(a, n_mats, n_groups, n_clusters, smem, s);
        default: return launch_bt<L, 8, false>(a, n_mats, n_groups, n_clusters, smem, s);
    }
}

}  // namespace

// n_mats same-shape, same-layout matrices with their own inputs and outputs in one launch.
// Inputs: xs[k] fp32 [N, ldx] with scales[k] = max|x| per token, or (half_in) xs[k] fp16 [N, ldx]
// already multiplied per token by a power of two with scales[k] = its inverse.  amax_outs
// (optional): [N] per matrix, merged with max|y| per token.
int launch_gemv_batch(const rwkvq_qtensor* ts, int n_mats, const void* const* xs, bool half_in, const float* const* scales,
                      int N, long long ldx, float* const* ys, long long ldy, int epilogue, const float* const* resids,
                      float* const* amax_outs, cudaStream_t s) {
    const int ml = mma_layout_of(ts[0]);
    RWKVQ_REQUIRE(ml >= 0, RWKVQ_E_DTYPE,
                  "rwkvq_gemv_batch: needs an sb6 tensor with relayouted records / planes, a sym tensor or per-row int8");
    RWKVQ_REQUIRE(n_mats >= 1 && n_mats <= kMmaMaxFused, RWKVQ_E_LIMIT, "rwkvq_gemv_batch: %d matrices", n_mats);
    BatchArgs a{};
    for (int k = 0; k < n_mats; ++k) {
        RWKVQ_REQUIRE(mma_layout_of(ts[k]) == ml && ts[k].rows == ts[0].rows && ts[k].cols == ts[0].cols, RWKVQ_E_SHAPE,
                      "rwkvq_gemv_batch: fused matrices must share layout and shape");
        RWKVQ_REQUIRE(xs[k] && ys[k] && scales[k], RWKVQ_E_NULL, "rwkvq_gemv_batch: x, its scales or y is null");
        RWKVQ_REQUIRE(aligned(xs[k], 16) && ldx % (half_in ? 8 : 4) == 0, RWKVQ_E_ALIGN,
                      "rwkvq_gemv_batch: x rows must be 16-byte aligned");
        a.t[k] = make_view(ts[k]);
        if (half_in) { a.x16[k] = static_cast<const __half*>(xs[k]); a.unscale[k] = scales[k]; }
        else { a.x[k] = static_cast<const float*>(xs[k]); a.amax[k] = scales[k]; }
        a.y[k] = ys[k]; a.resid[k] = resids ? resids[k] : nullptr;
        a.amax_out[k] = amax_outs ? amax_outs[k] : nullptr;
        RWKVQ_REQUIRE(epilogue != RWKVQ_EPI_ADD || a.resid[k], RWKVQ_E_NULL, "rwkvq_gemv_batch: resid is null");
    }
    a.ldx = ldx; a.ldy = ldy; a.n_tokens = N; a.epilogue = epilogue;
    a.trace = g_batch_trace;
    const int rows = ts[0].rows, cols = ts[0].cols;
    const bool exact = !half_in && !batch_fast();
    switch (ml) {
        case ML_SB6_4: return launch_bt_l<ML_SB6_4>(a, n_mats, rows, cols, N, exact, s);
        case ML_SB6_5: return launch_bt_l<ML_SB6_5>(a, n_mats, rows, cols, N, exact, s);
        case ML_SB6_6: return launch_bt_l<ML_SB6_6>(a, n_mats, rows, cols, N, exact, s);
        case ML_SYM6: return launch_bt_l<ML_SYM6>(a, n_mats, rows, cols, N, exact, s);
        case ML_RTN8: return launch_bt_l<ML_RTN8>(a, n_mats, rows, cols, N, exact, s);
        default: return launch_bt_l<ML_SYM8>(a, n_mats, rows, cols, N, exact, s);
    }
}

int launch_row_amax(const float* x, long long ldx, int cols, int N, float* amax, int* status, cudaStream_t s) {
    cudaError_t e = launch_pdl(row_amax_kernel, dim3(N), dim3(256), 0, s, x, ldx, cols, amax, status);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "row_amax: %s", cudaGetErrorString(e));
    return RWKVQ_OK;
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" void rwkvq_profiling_batch_trace(void* buf8, int force_ks) {
    g_batch_trace = static_cast<unsigned long long*>(buf8);
    g_batch_force_ks = force_ks;
    g_batch_force_rows = g_batch_force_cols = 0;
}
extern "C" void rwkvq_profiling_batch_fast(int fast) { g_batch_fast = fast < 0 ? -1 : (fast ? 1 : 0); }
extern "C" void rwkvq_profiling_batch_force(int force_ks, int rows, int cols) {
    g_batch_force_ks = force_ks;
    g_batch_force_rows = rows;
    g_batch_force_cols = cols;
}

// [status word, padded to 256 bytes][N floats: max|x| per row]
extern "C" size_t rwkvq_gemv_batch_workspace_bytes(int N) { return N > 0 ? 256 + ((static_cast<size_t>(N) * sizeof(float) + 255) / 256) * 256 : 0; }

extern "C" int rwkvq_gemv_batch(const rwkvq_qtensor* t, const float* x, int N, int64_t ldx, float* y, int64_t ldy,
                                int epilogue, const float* resid, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = validate_qtensor(t, "rwkvq_gemv_batch");
    if (rc) return rc;
    RWKVQ_REQUIRE(N >= 1, RWKVQ_E_SHAPE, "rwkvq_gemv_batch: N=%d", N);
    RWKVQ_REQUIRE(epilogue >= RWKVQ_EPI_NONE && epilogue <= RWKVQ_EPI_ADD, RWKVQ_E_DTYPE, "rwkvq_gemv_batch: epilogue %d", epilogue);
    RWKVQ_REQUIRE(ldx >= t->cols && ldy >= t->rows, RWKVQ_E_SHAPE, "rwkvq_gemv_batch: ldx %lld / ldy %lld", (long long)ldx, (long long)ldy);
    RWKVQ_REQUIRE(x && y, RWKVQ_E_NULL, "rwkvq_gemv_batch: x or y is null");
    // default: the two-term mma.sync kernel.  The tcgen05 kernel (single fp16 operands) serves more than
    // 32 rows in fast mode, tensors the mma.sync kernel has no layout for, and the profiling override.
    const bool tcb = tcb_enabled() && gemm_tcb_ok(*t) && ldx % 8 == 0 &&
                     ((batch_fast() && N > 32) || mma_layout_of(*t) < 0 || tcb_forced());
    RWKVQ_REQUIRE(tcb || mma_layout_of(*t) >= 0, RWKVQ_E_DTYPE,
                  "rwkvq_gemv_batch: needs an sb6 tensor, a sym tensor or per-row int8 with columns in multiples of 128");
    RWKVQ_REQUIRE(aligned(x, 16) && ldx % 4 == 0, RWKVQ_E_ALIGN, "rwkvq_gemv_batch: x rows must be 16-byte aligned");
    RWKVQ_REQUIRE(aligned(workspace, 16), RWKVQ_E_ALIGN, "rwkvq_gemv_batch: workspace must be 16-byte aligned");
    RWKVQ_REQUIRE(workspace && workspace_bytes >= rwkvq_gemv_batch_workspace_bytes(N), RWKVQ_E_LIMIT,
                  "rwkvq_gemv_batch: workspace of %zu bytes, %zu needed", workspace_bytes, rwkvq_gemv_batch_workspace_bytes(N));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int* status = static_cast<int*>(workspace);
    float* amax = reinterpret_cast<float*>(static_cast<char*>(workspace) + 256);
    rc = launch_row_amax(x, ldx, t->cols, N, amax, status, s);
    if (rc) return rc;
    const void* xs[1] = {x};
    const float* am[1] = {amax};
    float* ys[1] = {y};
    const float* rs[1] = {resid};
    rc = tcb ? launch_gemm_tcb(t, 1, xs, false, am, N, ldx, ys, ldy, epilogue, rs, nullptr, status, s, !batch_fast())
             : launch_gemv_batch(t, 1, xs, false, am, N, ldx, ys, ldy, epilogue, rs, nullptr, s);
    return rc ? rc : check_launch("rwkvq_gemv_batch");
}
