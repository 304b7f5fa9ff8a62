// Quantized linear for a small batch of right-hand sides (3..64 decode streams, short verify
// runs): every packed weight byte is read ONCE for the whole batch.
//
//     y[n, o] = epi( sum_c W[o, c] x[n, c] ),   n < N
//
// Where the single-vector kernel (rwkvq_gemv_mma.cuh) spends its MMA columns on digits of one
// activation vector, this kernel puts the tokens there: mma.sync.m16n8k16 (f16 x f16 -> f32)
// with the weights as the 16-row operand and 8 tokens per MMA.
//   * a warp owns 16 output rows; thread (g, t) streams the codes of rows g, g+8 for blocks
//     2t, 2t+1 of each group of 8 blocks with the same 128-bit loads from the file layout as
//     the single-vector kernel (load_frag), one group ("iteration") ahead;
//   * the codes become fp16 weights in registers, fp16(q*s + m): bytes -> halves by a byte
//     permute onto the exponent pattern of 1024, one subtract and one fused multiply-add per two
//     weights with the block scale / min, which ARE fp16 values by the codec's definition, so
//     the product is rounded once (the same operand precision as the prefill GEMM);
//   * which four k an MMA slot of a thread holds is free as long as both operands agree, so a
//     thread feeds its OWN block's weights (the block whose scale it decoded) and the
//     activations are staged in shared memory in exactly that order: per MMA step the 8 tokens
//     x 4 quad lanes x 4 halves of a warp form 256 contiguous bytes;
//   * activations arrive as fp32, are scaled per (token, staged chunk) by a power of two and
//     rounded to fp16 once; the scale is undone on the fp32 accumulators;
//   * the K loop is split over a thread-block CLUSTER (up to 8 CTAs): each CTA leaves its
//     partial tile in its shared memory and, after one cluster barrier, every CTA adds a
//     slice of the tile over all ranks through distributed shared memory in rank order
//     (deterministic, no global scratch, no atomics), applies the epilogue and stores.
// No wait in this kernel spins: the only synchronisation is the hardware cluster barrier.
#include <cooperative_groups.h>

#include <algorithm>

#include "rwkvq_gemv_mma.cuh"

namespace cg = cooperative_groups;

namespace rwkvq {

constexpr int kBtWarps = 8;
constexpr int kBtMaxChunkK = 512;        // columns of x staged at a time
constexpr int kBtStepPad = 16;           // bytes between MMA steps in shared memory (bank spread of the staging stores)

struct BatchArgs {
    QView t[kMmaMaxFused];
    const float* x[kMmaMaxFused];        // [N, ldx] per matrix
    float* y[kMmaMaxFused];              // [N, ldy]
    const float* resid[kMmaMaxFused];    // [N, ldy] or null
    long long ldx, ldy;
    int n_tokens;
    int epilogue;
    int tiles_per_cta;                   // 16-row tiles of one CTA
    int its_per_cta;                     // iterations (Geo::KI columns each) of one CTA's K slice
    int chunk_its;                       // iterations staged per shared-memory chunk
    int ks;                              // CTAs along K = cluster size
};

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

// Shared-memory order of the staged activations.  An iteration covers KI columns = 8 blocks;
// thread t of a quad owns blocks 2t + h.  MMA step s = ((h * NJ) + j) * 2 + half takes, from
// every quad lane, the 4 weights at offset koff(j, half) of its block, so element
// (token n, lane t, e < 4) of step s is x[n][it * KI + (2t + h) * BLK + koff + e].
template <int L> struct BtGeo {
    static constexpr int NJ = (L <= ML_SB6_6) ? 4 : 2;
    static constexpr int STEPS = Geo<L>::KI / 16;
    __device__ static constexpr int koff(int j, int half) { return (L <= ML_SB6_6) ? half * 16 + 4 * j : j * 8 + half * 4; }
};

template <int L, int NT, bool MC>      // NT: 8-token tiles; MC: the K slice of a CTA spans several staged chunks
__global__ void __launch_bounds__(kBtWarps * 32) gemv_batch_kernel(const BatchArgs a) {
    using G = Geo<L>;
    using BG = BtGeo<L>;
    constexpr int N8 = NT * 8;
    constexpr int SP = N8 * 32 + kBtStepPad;          // bytes per MMA step
    constexpr bool SB6 = L <= ML_SB6_6;
    extern __shared__ __align__(16) unsigned char smem[];
    cg::cluster_group cluster = cg::this_cluster();

    const QView& q = a.t[blockIdx.y];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int ks = a.ks, rank = static_cast<int>(blockIdx.x) % ks, rg = static_cast<int>(blockIdx.x) / ks;
    const int n0 = blockIdx.z * N8;                                     // first token of this CTA's group
    const int nn = min(N8, a.n_tokens - n0);
    const int R = a.tiles_per_cta * 16, RP = R + 4;
    const int n_tiles = (q.rows + 15) >> 4;
    const int tile0 = rg * a.tiles_per_cta;
    const int it_base = rank * a.its_per_cta;
    const int n_chunks = (a.its_per_cta + a.chunk_its - 1) / a.chunk_its;

    unsigned char* xs = smem;                                                           // staged fp16 activations
    float* unscale = reinterpret_cast<float*>(smem + static_cast<size_t>(a.chunk_its) * BG::STEPS * SP);
    float* part = unscale + N8;                                                         // [N8][RP] partial sums

    // this warp's tiles: warp, warp + 8, ...; flat item sequence (tile, iteration) for the prefetch
    const int my_tiles = (a.tiles_per_cta - warp + kBtWarps - 1) / kBtWarps;
    const int n_items = my_tiles * a.its_per_cta;
    int i_n = 0, i_tile = tile0 + warp, i_it = 0;
    Frag<L> nxt;
    auto fetch_next = [&]() {
        if (i_n < n_items && i_tile < n_tiles) {
            const int r0 = min(i_tile * 16 + g, q.rows - 1), r1 = min(i_tile * 16 + g + 8, q.rows - 1);
            load_frag<L>(nxt, q, r0, r1, it_base + i_it, t);
        }
        ++i_n;
        if (++i_it == a.its_per_cta) { i_it = 0; i_tile += kBtWarps; }
    };
    pdl_launch_dependents();
    fetch_next();                          // weights do not depend on the producer of x
    pdl_wait();

    const float* xg = a.x[blockIdx.y] + static_cast<size_t>(n0) * a.ldx;
    float tot[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) tot[i][0] = tot[i][1] = tot[i][2] = tot[i][3] = 0.f;
    const __half2 bias = __float2half2_rn(L == ML_SYM6 ? 1056.f : (L == ML_SYM8 || L == ML_RTN8) ? 1152.f : 1024.f);

    for (int ch = 0; ch < n_chunks; ++ch) {
        const int cits = min(a.chunk_its, a.its_per_cta - ch * a.chunk_its);
        const int kbase = (it_base + ch * a.chunk_its) * G::KI;
        const int f4_row = cits * G::KI / 4;                    // float4 per token in this chunk (<= 128)
        if (MC && ch > 0) __syncthreads();                      // everyone is done with the previous chunk
        // ---- stage: warp w takes tokens w, w + 8, ... in groups of 4 (loads of a group in flight together)
        for (int nb = warp; nb < N8; nb += 4 * kBtWarps) {
            float4 v[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int n = nb + u * kBtWarps;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int k4 = lane + 32 * i;
                    v[u][i] = (n < nn && k4 < f4_row)
                                  ? __ldcg(reinterpret_cast<const float4*>(xg + static_cast<size_t>(n) * a.ldx + kbase) + k4)
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int n = nb + u * kBtWarps;
                if (n >= N8) break;
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[u][i].x), fabsf(v[u][i].y)), fmaxf(fabsf(v[u][i].z), fabsf(v[u][i].w))));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
                // |x| * 2^(14 - e) <= 2^14 with amax <= 2^e; a non-finite row keeps scale 1 and propagates
                int e = 0;
                float sc = 1.f, un = 1.f;
                if (amax > 0.f && amax < INFINITY) {
                    frexpf(amax, &e);
                    e = max(-100, e);                       // 2^(14 - e) must stay finite
                    sc = ldexpf(1.f, 14 - e);
                    un = ldexpf(1.f, e - 14);
                }
                if (lane == 0) unscale[n] = un;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int k4 = lane + 32 * i;
                    if (k4 >= f4_row) break;
                    const int k = 4 * k4, it_l = k / G::KI, rem = k % G::KI;
                    const int blk = rem / G::BLK, off = rem % G::BLK;
                    const int tt = blk >> 1, h = blk & 1;
                    const int half = SB6 ? (off >> 4) : ((off >> 2) & 1), j = SB6 ? ((off >> 2) & 3) : (off >> 3);
                    const int step = it_l * BG::STEPS + ((h * BG::NJ) + j) * 2 + half;
                    const __half2 h01 = __floats2half2_rn(v[u][i].x * sc, v[u][i].y * sc);
                    const __half2 h23 = __floats2half2_rn(v[u][i].z * sc, v[u][i].w * sc);
                    uint2 pk;
                    pk.x = *reinterpret_cast<const uint32_t*>(&h01);
                    pk.y = *reinterpret_cast<const uint32_t*>(&h23);
                    *reinterpret_cast<uint2*>(xs + static_cast<size_t>(step) * SP + n * 32 + tt * 8) = pk;
                }
            }
        }
        __syncthreads();
        // ---- multiply: this warp's tiles over the staged iterations
        for (int ti = 0; ti < my_tiles; ++ti) {
            const int tile = tile0 + warp + ti * kBtWarps;
            float c[NT][4];
#pragma unroll
            for (int i = 0; i < NT; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
            for (int il = 0; il < cits; ++il) {
                const Frag<L> cur = nxt;
                fetch_next();
                if (tile >= n_tiles) continue;
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
                const unsigned char* xrow = xs + static_cast<size_t>(il) * BG::STEPS * SP + g * 32 + t * 8;
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
            // chunk done for this tile: undo the per-token scale (C columns 2t, 2t+1 of each 8-token tile)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float u0 = unscale[nt * 8 + 2 * t], u1 = unscale[nt * 8 + 2 * t + 1];
                if (MC) {
                    tot[nt][0] = fmaf(c[nt][0], u0, tot[nt][0]); tot[nt][1] = fmaf(c[nt][1], u1, tot[nt][1]);
                    tot[nt][2] = fmaf(c[nt][2], u0, tot[nt][2]); tot[nt][3] = fmaf(c[nt][3], u1, tot[nt][3]);
                } else {
                    tot[nt][0] = c[nt][0] * u0; tot[nt][1] = c[nt][1] * u1;
                    tot[nt][2] = c[nt][2] * u0; tot[nt][3] = c[nt][3] * u1;
                }
            }
            if (!MC || ch == n_chunks - 1) {
                const int r = (warp + ti * kBtWarps) * 16 + g;          // row inside the CTA's group
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int n = nt * 8 + 2 * t;
                    part[n * RP + r] = tot[nt][0];
                    part[(n + 1) * RP + r] = tot[nt][1];
                    part[n * RP + r + 8] = tot[nt][2];
                    part[(n + 1) * RP + r + 8] = tot[nt][3];
                }
            }
        }
    }
    // ---- add the K slices of the cluster in rank order, epilogue, store
    cluster.sync();
    {
        const int total = nn * R;
        const int per = (total + ks - 1) / ks;
        const int lo = rank * per, hi = min(total, lo + per);
        const int row0 = rg * R;
        float* y = a.y[blockIdx.y] + static_cast<size_t>(n0) * a.ldy;
        const float* resid = a.resid[blockIdx.y] ? a.resid[blockIdx.y] + static_cast<size_t>(n0) * a.ldy : nullptr;
        for (int idx = lo + threadIdx.x; idx < hi; idx += kBtWarps * 32) {
            const int n = idx / R, r = idx - n * R;
            const int row = row0 + r;
            if (row >= q.rows) continue;
            float v = 0.f;
            for (int k = 0; k < ks; ++k) v += cluster.map_shared_rank(part, k)[n * RP + r];
            const size_t o = static_cast<size_t>(n) * a.ldy + row;
            if (a.epilogue == RWKVQ_EPI_RELU2) { v = fmaxf(v, 0.f); v = v * v; }
            else if (a.epilogue == RWKVQ_EPI_ADD) v = __fadd_rn(v, __ldcg(resid + o));
            y[o] = v;
        }
    }
    cluster.sync();          // nobody leaves while a peer still reads its partial tile
}

namespace {

constexpr int kBtMaxSmem = 200 * 1024;

template <int L, int NT, bool MC>
int launch_bt(BatchArgs& a, int n_mats, int n_groups, int row_groups, size_t smem, cudaStream_t s) {
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
    if (dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_batch_kernel<L, NT, MC>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBtMaxSmem);
        if (e != cudaSuccess) return fail(RWKVQ_E_LIMIT, "rwkvq_gemv_batch: shared memory attribute: %s", cudaGetErrorString(e));
        if (dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(row_groups * a.ks, n_mats, n_groups);
    cfg.blockDim = dim3(kBtWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = a.ks; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, gemv_batch_kernel<L, NT, MC>, a);
    if (le != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_gemv_batch: %s", cudaGetErrorString(le));
    return RWKVQ_OK;
}

template <int L>
int launch_bt_l(BatchArgs& a, int n_mats, int rows, int cols, int N, cudaStream_t s) {
    using G = Geo<L>;
    const int n_iters = cols / G::KI;
    int ks = 1;
    for (int c = 8; c > 1; --c)
        if (n_iters % c == 0) { ks = c; break; }
    a.ks = ks;
    a.its_per_cta = n_iters / ks;
    a.chunk_its = std::min(a.its_per_cta, kBtMaxChunkK / G::KI);
    const bool mc = a.its_per_cta > a.chunk_its;
    const int nt = N <= 8 ? 1 : N <= 16 ? 2 : N <= 32 ? 4 : 8;
    const int n8 = nt * 8, n_groups = (N + n8 - 1) / n8;
    const int n_tiles = (rows + 15) / 16;
    // rows per CTA: 8 tiles (one per warp); more (the warps loop) while the grid would exceed two
    // waves of resident CTAs and the partial tile still fits; fewer for short matrices
    int tpc = std::min(8, n_tiles);
    if (!mc)
        while (tpc < 32 && ((n_tiles + tpc - 1) / tpc) * ks * n_mats * n_groups > 2 * 148) tpc *= 2;
    a.tiles_per_cta = tpc;
    const int row_groups = (n_tiles + tpc - 1) / tpc;
    const size_t smem = static_cast<size_t>(a.chunk_its) * (G::KI / 16) * (n8 * 32 + kBtStepPad) + n8 * sizeof(float) +
                        static_cast<size_t>(n8) * (tpc * 16 + 4) * sizeof(float);
    if (smem > static_cast<size_t>(kBtMaxSmem)) return fail(RWKVQ_E_LIMIT, "rwkvq_gemv_batch: %zu bytes of shared memory", smem);
#define RWKVQ_BT(NTV)                                                                                  \
    return mc ? launch_bt<L, NTV, true>(a, n_mats, n_groups, row_groups, smem, s)                       \
              : launch_bt<L, NTV, false>(a, n_mats, n_groups, row_groups, smem, s)
    switch (nt) {
        case 1: RWKVQ_BT(1);
        case 2: RWKVQ_BT(2);
        case 4: RWKVQ_BT(4);
        default: RWKVQ_BT(8);
    }
#undef RWKVQ_BT
}

}  // namespace

// n_mats same-shape, same-layout matrices with their own inputs and outputs in one launch.
int launch_gemv_batch(const rwkvq_qtensor* ts, int n_mats, const float* const* xs, int N, long long ldx,
                      float* const* ys, long long ldy, int epilogue, const float* const* resids, cudaStream_t s) {
    const int ml = mma_layout_of(ts[0]);
    RWKVQ_REQUIRE(ml >= 0, RWKVQ_E_DTYPE,
                  "rwkvq_gemv_batch: needs an sb6 tensor with relayouted records / planes, a sym tensor or per-row int8");
    RWKVQ_REQUIRE(n_mats >= 1 && n_mats <= kMmaMaxFused, RWKVQ_E_LIMIT, "rwkvq_gemv_batch: %d matrices", n_mats);
    BatchArgs a{};
    for (int k = 0; k < n_mats; ++k) {
        RWKVQ_REQUIRE(mma_layout_of(ts[k]) == ml && ts[k].rows == ts[0].rows && ts[k].cols == ts[0].cols, RWKVQ_E_SHAPE,
                      "rwkvq_gemv_batch: fused matrices must share layout and shape");
        RWKVQ_REQUIRE(xs[k] && ys[k], RWKVQ_E_NULL, "rwkvq_gemv_batch: x or y is null");
        RWKVQ_REQUIRE(aligned(xs[k], 16) && ldx % 4 == 0, RWKVQ_E_ALIGN, "rwkvq_gemv_batch: x rows must be 16-byte aligned");
        a.t[k] = make_view(ts[k]);
        a.x[k] = xs[k]; a.y[k] = ys[k]; a.resid[k] = resids ? resids[k] : nullptr;
        RWKVQ_REQUIRE(epilogue != RWKVQ_EPI_ADD || a.resid[k], RWKVQ_E_NULL, "rwkvq_gemv_batch: resid is null");
    }
    a.ldx = ldx; a.ldy = ldy; a.n_tokens = N; a.epilogue = epilogue;
    const int rows = ts[0].rows, cols = ts[0].cols;
    switch (ml) {
        case ML_SB6_4: return launch_bt_l<ML_SB6_4>(a, n_mats, rows, cols, N, s);
        case ML_SB6_5: return launch_bt_l<ML_SB6_5>(a, n_mats, rows, cols, N, s);
        case ML_SB6_6: return launch_bt_l<ML_SB6_6>(a, n_mats, rows, cols, N, s);
        case ML_SYM6: return launch_bt_l<ML_SYM6>(a, n_mats, rows, cols, N, s);
        case ML_RTN8: return launch_bt_l<ML_RTN8>(a, n_mats, rows, cols, N, s);
        default: return launch_bt_l<ML_SYM8>(a, n_mats, rows, cols, N, s);
    }
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" int rwkvq_gemv_batch(const rwkvq_qtensor* t, const float* x, int N, int64_t ldx, float* y, int64_t ldy,
                                int epilogue, const float* resid, void* stream) {
    int rc = validate_qtensor(t, "rwkvq_gemv_batch");
    if (rc) return rc;
    RWKVQ_REQUIRE(N >= 1, RWKVQ_E_SHAPE, "rwkvq_gemv_batch: N=%d", N);
    RWKVQ_REQUIRE(epilogue >= RWKVQ_EPI_NONE && epilogue <= RWKVQ_EPI_ADD, RWKVQ_E_DTYPE, "rwkvq_gemv_batch: epilogue %d", epilogue);
    RWKVQ_REQUIRE(ldx >= t->cols && ldy >= t->rows, RWKVQ_E_SHAPE, "rwkvq_gemv_batch: ldx %lld / ldy %lld", (long long)ldx, (long long)ldy);
    const float* xs[1] = {x};
    float* ys[1] = {y};
    const float* rs[1] = {resid};
    rc = launch_gemv_batch(t, 1, xs, N, ldx, ys, ldy, epilogue, rs, static_cast<cudaStream_t>(stream));
    return rc ? rc : check_launch("rwkvq_gemv_batch");
}
