// Single-vector decode GEMV on the integer tensor-core path.
//
// The codes of the .rwkvq layouts are small integers, so the inner products
// sum_c q_c * X_c are computed EXACTLY in int32 by mma.sync.m16n8k32 (u8/s8 x s8):
//   * the activation vector is turned once per CTA into a 21-bit fixed-point
//     vector X = round(x * 2^e) (2^e chosen from max|x|) and split into three
//     signed 7-bit digits  X = d1*2^14 + d2*2^7 + d3  kept in shared memory;
//   * a warp owns 16 output rows; thread (g, t) of the warp streams the codes of
//     rows g and g+8 for blocks 2t and 2t+1 of each group of 8 blocks with
//     128-bit loads straight from the file layout (a quad reads 128 contiguous
//     bytes of a row), turns nibbles into bytes with one AND per 4 weights and
//     feeds them to the MMA as the A operand;
//   * the 8 MMA columns are (block of the quad lane, digit): the B operand of
//     column 2t+dg is digit dg of the activations of thread t's block and zero
//     elsewhere, so C[row, 2t+dg] is the integer dot product of (row, block)
//     with digit dg and every thread ends up holding the dot products of exactly
//     the (row, block) pairs whose scale codes it loaded;
//   * the per-block scale s = fp16(qs*d) (and min) is applied in fp32 per block,
//     which is the arithmetic the codec defines; accumulation over blocks is fp32.
// No dequantised copy of the weights ever exists; the only approximation is the
// 21-bit fixed-point activation (relative error <= 2^-20 of max|x| per element).
#include "rwkvq_common.cuh"

namespace rwkvq {

enum MmaLayout { ML_SB6_4 = 0, ML_SB6_5, ML_SB6_6, ML_SYM6, ML_SYM8 };

constexpr int kMmaWarps = 8;
constexpr int kMmaMaxFused = 4;

struct MmaArgs {
    QView t[kMmaMaxFused];
    const void* x;      // [n_mats, ldx] (fused) or [ldx]
    const void* xk[kMmaMaxFused];   // optional per-matrix inputs (fused launches with scattered rows)
    int x_dtype;
    long long ldx;
    float* y;
    long long ldy;
    const float* resid;
    int epilogue;
    int fused;
    // split of the K loop over gridDim.z CTAs: partial row sums go to `partial`
    // [gridDim.z][n_mats][rows_padded] and the last CTA of a tile group to arrive
    // (counted in `counters`, which it resets) adds them in slice order
    float* partial;
    unsigned int* counters;
    int rows_padded;
};

template <bool A_UNSIGNED>
__device__ __forceinline__ void mma_i8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    if (A_UNSIGNED) {
        asm volatile(
            "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

template <int L> struct Geo;   // K per iteration, bytes of codes per (row, thread, iteration)
template <> struct Geo<ML_SB6_4> { static constexpr int KI = 256, BLK = 32, BITS = 4; };
template <> struct Geo<ML_SB6_5> { static constexpr int KI = 256, BLK = 32, BITS = 5; };
template <> struct Geo<ML_SB6_6> { static constexpr int KI = 256, BLK = 32, BITS = 6; };
template <> struct Geo<ML_SYM6> { static constexpr int KI = 128, BLK = 16, BITS = 6; };
template <> struct Geo<ML_SYM8> { static constexpr int KI = 128, BLK = 16, BITS = 8; };

// Everything thread (g, t) streams for one iteration (8 blocks) of rows g, g+8.
template <int L>
struct Frag {
    uint4 ca[2], cb[2];    // codes of blocks 2t, 2t+1: row g (ca), row g+8 (cb)
    uint4 ma, mb;          // sb6: 16-byte scale records;  sym: .x,.y = 8 scale codes, .z = d bits
    uint4 pa, pb;          // regrouped bit-planes of the two blocks
};

// sb6 scale record (16 bytes per row and super-block, written by rwkvq_relayout_meta):
// word t (t = 0..3) serves the thread that owns blocks 2t and 2t+1:
//   bits  0-5  qs[2t]      bits  6-11 qs[2t+1]        (6-bit scale codes)
//   bits 12-17 qm[2t]+31   bits 18-23 qm[2t+1]+31     (6-bit min codes as stored)
//   bits 24-31 byte t of the 32-bit value (d | dm << 16) (the two fp16 super-scales)
// Returns (s0, s1) and (m0, m1) of the two blocks: s = max(fp16(qs*d), 1e-8),
// m = fp16(qm*dm).  A half-precision multiply of the exact small integer by the
// fp16 super-scale rounds the exact product once, which is the codec's definition.
__device__ __forceinline__ void sb6_pair_scales(const uint4& rec, int t, float2& s, float2& m) {
    const uint32_t w = (t & 2) ? ((t & 1) ? rec.w : rec.z) : ((t & 1) ? rec.y : rec.x);
    const uint32_t dd = __byte_perm(rec.x, rec.y, 0x7373);     // half2(d, d)
    const uint32_t dmm = __byte_perm(rec.z, rec.w, 0x7373);    // half2(dm, dm)
    // 1024 + code as fp16 bits, two codes per register
    const uint32_t qs = (w & 0x3Fu) | ((w << 10) & 0x003F0000u) | 0x64006400u;
    const uint32_t qm = ((w >> 12) & 0x3Fu) | ((w >> 2) & 0x003F0000u) | 0x64006400u;
    const __half2 hs = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&qs), __float2half2_rn(1024.f)),
                               *reinterpret_cast<const __half2*>(&dd));
    const __half2 hm = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&qm), __float2half2_rn(1055.f)),
                               *reinterpret_cast<const __half2*>(&dmm));
    s = __half22float2(hs);
    m = __half22float2(hm);
    s.x = fmaxf(s.x, 1e-8f);
    s.y = fmaxf(s.y, 1e-8f);
}

// sym: the two int8 scale codes of blocks 2t, 2t+1 times the fp16 super-scale
__device__ __forceinline__ float2 sym_pair_scales(uint32_t q_lo, uint32_t q_hi, uint32_t d_bits, int t) {
    const uint32_t w = (t & 2) ? q_hi : q_lo;
    const uint32_t two = (t & 1) ? (w >> 16) : (w & 0xFFFFu);          // bytes 2t, 2t+1
    // (code + 128) + 1024 as fp16 bits
    const uint32_t u = ((two ^ 0x8080u) & 0xFFu) | (((two ^ 0x8080u) << 8) & 0x00FF0000u) | 0x64006400u;
    const uint32_t dd = d_bits | (d_bits << 16);
    const __half2 hs = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&u), __float2half2_rn(1152.f)),
                               *reinterpret_cast<const __half2*>(&dd));
    return __half22float2(hs);
}

// Direct (register) loads of iteration `it` of rows r0, r1 for thread t.
template <int L>
__device__ __forceinline__ void load_frag(Frag<L>& f, const QView& q, int r0, int r1, int it, int t) {
    const size_t R0 = static_cast<size_t>(r0), R1 = static_cast<size_t>(r1);
    if (L <= ML_SB6_6) {
        const int nsb = q.cols >> 8;
        const size_t rowb = static_cast<size_t>(q.cols >> 1), nb = static_cast<size_t>(q.cols >> 5);
        const uint8_t* p0 = q.codes + R0 * rowb + it * 128 + t * 32;
        const uint8_t* p1 = q.codes + R1 * rowb + it * 128 + t * 32;
        f.ca[0] = ld_stream_u128(p0); f.ca[1] = ld_stream_u128(p0 + 16);
        f.cb[0] = ld_stream_u128(p1); f.cb[1] = ld_stream_u128(p1 + 16);
        f.ma = ld_stream_u128(q.dev_meta + (R0 * nsb + it) * 16);
        f.mb = ld_stream_u128(q.dev_meta + (R1 * nsb + it) * 16);
        if (L == ML_SB6_5) {
            const uint2 a = ld_stream_u64(q.dev_planes + R0 * nb + it * 8 + 2 * t);
            const uint2 b = ld_stream_u64(q.dev_planes + R1 * nb + it * 8 + 2 * t);
            f.pa = make_uint4(a.x, a.y, 0, 0); f.pb = make_uint4(b.x, b.y, 0, 0);
        } else if (L == ML_SB6_6) {
            f.pa = ld_stream_u128(q.dev_planes + (R0 * nb + it * 8 + 2 * t) * 2);
            f.pb = ld_stream_u128(q.dev_planes + (R1 * nb + it * 8 + 2 * t) * 2);
        }
    } else {
        const size_t nb16 = static_cast<size_t>(q.cols >> 4);
        const int nsb = q.cols >> 8;
        if (L == ML_SYM6) {
            const size_t rowb = static_cast<size_t>(q.cols >> 1);
            f.ca[0] = ld_stream_u128(q.codes + R0 * rowb + it * 64 + t * 16);
            f.cb[0] = ld_stream_u128(q.codes + R1 * rowb + it * 64 + t * 16);
            const uint2 a = ld_stream_u64(q.dev_planes + R0 * nb16 + it * 8 + 2 * t);
            const uint2 b = ld_stream_u64(q.dev_planes + R1 * nb16 + it * 8 + 2 * t);
            f.pa = make_uint4(a.x, a.y, 0, 0); f.pb = make_uint4(b.x, b.y, 0, 0);
        } else {
            const size_t rowb = static_cast<size_t>(q.cols);
            const uint8_t* p0 = q.codes + R0 * rowb + it * 128 + t * 32;
            const uint8_t* p1 = q.codes + R1 * rowb + it * 128 + t * 32;
            f.ca[0] = ld_stream_u128(p0); f.ca[1] = ld_stream_u128(p0 + 16);
            f.cb[0] = ld_stream_u128(p1); f.cb[1] = ld_stream_u128(p1 + 16);
        }
        const uint2 sa = ld_stream_u64(reinterpret_cast<const uint8_t*>(q.qs) + R0 * nb16 + it * 8);
        const uint2 sb = ld_stream_u64(reinterpret_cast<const uint8_t*>(q.qs) + R1 * nb16 + it * 8);
        f.ma = make_uint4(sa.x, sa.y, ld_stream_u16(q.d + R0 * nsb + (it >> 1)), 0);
        f.mb = make_uint4(sb.x, sb.y, ld_stream_u16(q.d + R1 * nsb + (it >> 1)), 0);
    }
}

__device__ __forceinline__ uint32_t word_of(const uint4& v, int j) {
    return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w;
}

// A-operand words of block h (0/1 of the thread's pair): for MMA step j the
// low-half word (weights in K slots 4t..4t+3) and the high-half word (slots
// 16+4t..).  `pl` holds the regrouped planes of this block.
template <int L>
__device__ __forceinline__ void a_words(const uint4 (&c)[2], const uint4& planes, int h, int j,
                                        uint32_t& lo, uint32_t& hi) {
    using G = Geo<L>;
    if (L <= ML_SB6_6) {
        const uint32_t w = word_of(c[h], j);
        lo = w & 0x0F0F0F0Fu;
        hi = (w >> 4) & 0x0F0F0F0Fu;
        if (G::BITS == 5) {
            // plane word: bit (8b + G) = code bit 4 of weight (G < 4 ? 4G + b : 16 + 4(G-4) + b)
            const uint32_t p = h ? planes.y : planes.x;
            lo |= (p << (4 - j)) & 0x10101010u;
            hi |= (p >> j) & 0x10101010u;
        } else if (G::BITS == 6) {
            // two words per block: bits (8b + 2j, 8b + 2j + 1) = code bits (4, 5) of weight
            // 4j + b (first word) / 16 + 4j + b (second word)
            const uint32_t p0 = h ? planes.z : planes.x, p1 = h ? planes.w : planes.y;
            lo |= (j < 2 ? (p0 << (4 - 2 * j)) : (p0 >> (2 * j - 4))) & 0x30303030u;
            hi |= (j < 2 ? (p1 << (4 - 2 * j)) : (p1 >> (2 * j - 4))) & 0x30303030u;
        }
    } else if (L == ML_SYM6) {
        // block of 16: two code words; step 0 takes the low nibbles (weights 0-3, 4-7),
        // step 1 the high nibbles (weights 8-11, 12-15).  Plane word: bits
        // (8b + 2G, 8b + 2G + 1) = code bits (4, 5) of weight (G < 2 ? 4G + b : 8 + 4(G-2) + b)
        const uint32_t w0 = h ? c[0].z : c[0].x, w1 = h ? c[0].w : c[0].y;
        const uint32_t p = h ? planes.y : planes.x;
        if (j == 0) {
            lo = (w0 & 0x0F0F0F0Fu) | ((p << 4) & 0x30303030u);
            hi = (w1 & 0x0F0F0F0Fu) | ((p << 2) & 0x30303030u);
        } else {
            lo = ((w0 >> 4) & 0x0F0F0F0Fu) | (p & 0x30303030u);
            hi = ((w1 >> 4) & 0x0F0F0F0Fu) | ((p >> 2) & 0x30303030u);
        }
    } else {
        lo = word_of(c[h], 2 * j);
        hi = word_of(c[h], 2 * j + 1);
    }
}

// Activation -> fixed point digits in shared memory.
//   dig[d][i]  signed 7-bit digit d (0: most significant) of X_i = round(x_i * 2^e)
//   xs16[k]    sum of X over elements 16k..16k+15 (exact, as float)
// Returns 2^-e (the factor that undoes the scaling) and whether x was finite.
__device__ __forceinline__ float4 load_x4(const void* x, int dtype, int i) {
    // L2-coherent loads: under programmatic dependent launch this kernel is resident
    // while its producer still writes x, so the L1 / read-only path must not be used
    if (dtype == RWKVQ_F32) return __ldcg(reinterpret_cast<const float4*>(x) + i);
    const uint2 v = __ldcg(reinterpret_cast<const uint2*>(x) + i);
    if (dtype == RWKVQ_F16) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xFFFF0000u),
                       __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xFFFF0000u));
}

__device__ __forceinline__ void split_digits(int X, int& d1, int& d2, int& d3) {
    d3 = ((X + 64) & 127) - 64;
    const int x1 = (X - d3) >> 7;
    d2 = ((x1 + 64) & 127) - 64;
    d1 = (x1 - d2) >> 7;
}

// `bits` = 20 (|X| <= 2^20) or 19: chosen so that |sum over one block of q*X| < 2^31.
// x is read once: up to kXRegs float4 per thread stay in registers between the max
// pass and the conversion pass (IN <= 8192 at 256 threads); longer vectors are re-read.
constexpr int kXRegs = 8;
__device__ __forceinline__ float prepare_x(const void* x, int dtype, int n_in, int bits, int8_t* dig,
                                           float* xs16, float* red, bool& finite) {
    const int tid = threadIdx.x, n4 = n_in >> 2, nt = blockDim.x;
    float4 xr[kXRegs];
    float amax = 0.f;
    auto upd = [&](const float4& v) {
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        if (!(fabsf(v.x) + fabsf(v.y) + fabsf(v.z) + fabsf(v.w) < INFINITY)) amax = INFINITY;
    };
#pragma unroll
    for (int k = 0; k < kXRegs; ++k) {
        const int i = tid + k * nt;
        xr[k] = i < n4 ? load_x4(x, dtype, i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < kXRegs; ++k) upd(xr[k]);
    for (int i = tid + kXRegs * nt; i < n4; i += nt) upd(load_x4(x, dtype, i));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if ((tid & 31) == 0) red[tid >> 5] = amax;
    __syncthreads();
    amax = 0.f;
    for (int w = 0; w < (nt >> 5); ++w) amax = fmaxf(amax, red[w]);
    finite = amax < INFINITY;
    int e = 0;
    if (finite && amax > 0.f) frexpf(amax, &e);          // amax <= 2^e
    const float scale = finite ? ldexpf(1.f, bits - e) : 0.f;
    auto emit = [&](int i, const float4& v) {
        const int X0 = __float2int_rn(v.x * scale), X1 = __float2int_rn(v.y * scale);
        const int X2 = __float2int_rn(v.z * scale), X3 = __float2int_rn(v.w * scale);
        int a[4], b[4], c[4];
        split_digits(X0, a[0], b[0], c[0]); split_digits(X1, a[1], b[1], c[1]);
        split_digits(X2, a[2], b[2], c[2]); split_digits(X3, a[3], b[3], c[3]);
        auto pack = [](const int (&d)[4]) {
            return (d[0] & 0xFF) | ((d[1] & 0xFF) << 8) | ((d[2] & 0xFF) << 16) | (static_cast<uint32_t>(d[3] & 0xFF) << 24);
        };
        reinterpret_cast<uint32_t*>(dig)[i] = pack(a);
        reinterpret_cast<uint32_t*>(dig + n_in)[i] = pack(b);
        reinterpret_cast<uint32_t*>(dig + 2 * n_in)[i] = pack(c);
        int s = X0 + X1 + X2 + X3;        // the 4 lanes of an aligned quad cover one 16-chunk
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
        if ((tid & 3) == 0) xs16[i >> 2] = static_cast<float>(s);
    };
#pragma unroll
    for (int k = 0; k < kXRegs; ++k) {
        const int i = tid + k * nt;
        if (i < n4) emit(i, xr[k]);          // n4 is a multiple of 64: whole warps take this branch together
    }
    for (int i = tid + kXRegs * nt; i < n4; i += nt) emit(i, load_x4(x, dtype, i));
    __syncthreads();
    return finite ? ldexpf(1.f, e - bits) : 0.f;
}

// Persistent kernel: gridDim.x CTAs walk the 16-row tiles of matrix blockIdx.y with
// stride gridDim.x * WT.  Inside a CTA step the 8 warps form WT tiles x WK slices
// of the K loop; the activations are prepared once per CTA.  Each warp sees a flat
// sequence of work items (tile, iteration); the loads of item n+1 are issued
// before item n is consumed.
template <int L, int WK>
__global__ void __launch_bounds__(kMmaWarps * 32, 2) gemv_mma_kernel(const MmaArgs a) {
    using G = Geo<L>;
    constexpr int WT = kMmaWarps / WK;
    constexpr bool SB6 = L <= ML_SB6_6;
    constexpr bool A_UNSIGNED = L != ML_SYM8;
    extern __shared__ __align__(16) unsigned char smem[];
    const QView& q = a.t[blockIdx.y];
    const int n_in = q.cols;
    int8_t* dig = reinterpret_cast<int8_t*>(smem);
    float* xs16 = reinterpret_cast<float*>(dig + 3 * n_in);
    float* red = xs16 + (n_in >> 4);                                     // [2][kMmaWarps * 16]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int tl = warp / WK, ks = warp % WK;
    const int KS = gridDim.z;                               // K slices across CTAs
    const int n_iters = n_in / G::KI / KS;                  // iterations of this CTA's slice
    const int it0 = blockIdx.z * n_iters;
    const int n_tiles = (q.rows + 15) >> 4;
    const int step = gridDim.x * WT;
    const int ipt = (n_iters - ks + WK - 1) / WK;          // this warp's iterations per tile
    const int n_steps = ((n_tiles + WT - 1) / WT - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                        static_cast<int>(gridDim.x);
    const int n_items = n_steps * ipt;
    // prefetch side: item counter -> (tile, iteration)
    int i_n = 0, i_tile = blockIdx.x * WT + tl, i_j = 0;
    Frag<L> nxt;
    auto fetch_next = [&]() {
        if (i_n < n_items && i_tile < n_tiles) {
            const int r0 = min(i_tile * 16 + g, q.rows - 1), r1 = min(i_tile * 16 + g + 8, q.rows - 1);
            load_frag<L>(nxt, q, r0, r1, it0 + ks + i_j * WK, t);
        }
        ++i_n;
        if (++i_j == ipt) { i_j = 0; i_tile += step; }
    };
    // the first weight loads go out before the activations are touched (and before the
    // producer of the activations has finished, when launched programmatically)
    pdl_launch_dependents();
    fetch_next();
    pdl_wait();

    const size_t esz = (a.x_dtype == RWKVQ_F32) ? 4 : 2;
    const char* xv = a.xk[blockIdx.y] ? static_cast<const char*>(a.xk[blockIdx.y])
                                      : static_cast<const char*>(a.x) + (a.fused ? blockIdx.y * a.ldx * esz : 0);
    bool finite;
    const float unscale = prepare_x(xv, a.x_dtype, n_in, L == ML_SYM8 ? 19 : 20, dig, xs16, red, finite);
    __syncthreads();

    // which B columns this lane feeds: column 2t+dg of MMA set 1, column 2t of set 2
    const bool b_set1 = (g >> 1) == t;
    const bool b_set2 = g == 2 * t;
    const int8_t* dig1 = dig + (g & 1) * n_in;
    const int8_t* dig3 = dig + 2 * n_in;

    int c_n = 0, buf = 0;
    for (int base = blockIdx.x * WT; base < n_tiles; base += step, buf ^= 1) {
        const int tile = base + tl;
        float acc0 = 0.f, acc1 = 0.f;     // rows g, g+8 of this tile
        for (int j = 0; j < ipt; ++j, ++c_n) {
            const Frag<L> cur = nxt;
            fetch_next();
            if (tile >= n_tiles) continue;
            const int it = it0 + ks + j * WK;

            float2 sa, sb, ma = make_float2(0.f, 0.f), mb = ma;
            if (SB6) {
                sb6_pair_scales(cur.ma, t, sa, ma);
                sb6_pair_scales(cur.mb, t, sb, mb);
            } else {
                sa = sym_pair_scales(cur.ma.x, cur.ma.y, cur.ma.z, t);
                sb = sym_pair_scales(cur.mb.x, cur.mb.y, cur.mb.z, t);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int blk = it * 8 + 2 * t + h;            // block index along the row
                int c[4] = {0, 0, 0, 0}, e[4] = {0, 0, 0, 0};
                if (SB6) {
                    uint4 b1lo = make_uint4(0, 0, 0, 0), b1hi = b1lo, b3lo = b1lo, b3hi = b1lo;
                    if (b_set1) {
                        b1lo = *reinterpret_cast<const uint4*>(dig1 + blk * 32);
                        b1hi = *reinterpret_cast<const uint4*>(dig1 + blk * 32 + 16);
                    }
                    if (b_set2) {
                        b3lo = *reinterpret_cast<const uint4*>(dig3 + blk * 32);
                        b3hi = *reinterpret_cast<const uint4*>(dig3 + blk * 32 + 16);
                    }
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        uint32_t a0, a1, a2, a3;
                        a_words<L>(cur.ca, cur.pa, h, jj, a0, a2);
                        a_words<L>(cur.cb, cur.pb, h, jj, a1, a3);
                        mma_i8<A_UNSIGNED>(c, a0, a1, a2, a3, word_of(b1lo, jj), word_of(b1hi, jj));
                        mma_i8<A_UNSIGNED>(e, a0, a1, a2, a3, word_of(b3lo, jj), word_of(b3hi, jj));
                    }
                } else {
                    uint4 b1 = make_uint4(0, 0, 0, 0), b3 = b1;
                    if (b_set1) b1 = *reinterpret_cast<const uint4*>(dig1 + blk * 16);
                    if (b_set2) b3 = *reinterpret_cast<const uint4*>(dig3 + blk * 16);
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) {
                        uint32_t a0, a1, a2, a3;
                        a_words<L>(cur.ca, cur.pa, h, jj, a0, a2);
                        a_words<L>(cur.cb, cur.pb, h, jj, a1, a3);
                        mma_i8<A_UNSIGNED>(c, a0, a1, a2, a3, word_of(b1, 2 * jj), word_of(b1, 2 * jj + 1));
                        mma_i8<A_UNSIGNED>(e, a0, a1, a2, a3, word_of(b3, 2 * jj), word_of(b3, 2 * jj + 1));
                    }
                }
                // c[0], c[1]: row g digits 1, 2;  c[2], c[3]: row g+8;  e[0], e[2]: digit 3.
                // The recombined value is the exact integer sum q*X of the block (< 2^31).
                const float f0 = static_cast<float>((c[0] << 14) + (c[1] << 7) + e[0]);
                const float f1 = static_cast<float>((c[2] << 14) + (c[3] << 7) + e[2]);
                const float s0 = h ? sa.y : sa.x, s1 = h ? sb.y : sb.x;
                if (SB6) {
                    const float xsum = xs16[2 * blk] + xs16[2 * blk + 1];
                    acc0 = fmaf(s0, f0, fmaf(h ? ma.y : ma.x, xsum, acc0));
                    acc1 = fmaf(s1, f1, fmaf(h ? mb.y : mb.x, xsum, acc1));
                } else {
                    const float off = (L == ML_SYM6) ? -32.f * xs16[blk] : 0.f;   // codes are stored +32
                    acc0 = fmaf(s0, f0 + off, acc0);
                    acc1 = fmaf(s1, f1 + off, acc1);
                }
            }
        }
        // the 4 lanes of a quad hold the 8 blocks of each iteration
        acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 1); acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 2);
        acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 1); acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 2);
        float* rb = red + buf * (kMmaWarps * 16);
        if (t == 0) { rb[warp * 16 + g] = acc0; rb[warp * 16 + g + 8] = acc1; }
        __syncthreads();
        if (KS == 1) {
            if (threadIdx.x < WT * 16) {
                const int wtl = threadIdx.x >> 4, r = threadIdx.x & 15;
                const int row = (base + wtl) * 16 + r;
                if (row < q.rows) {
                    float v = 0.f;
#pragma unroll
                    for (int k = 0; k < WK; ++k) v += rb[(wtl * WK + k) * 16 + r];
                    v = finite ? v * unscale : NAN;
                    const long long idx = (a.fused ? static_cast<long long>(blockIdx.y) * a.ldy : 0) + row;
                    if (a.epilogue == RWKVQ_EPI_RELU2) { v = fmaxf(v, 0.f); v = v * v; }
                    else if (a.epilogue == RWKVQ_EPI_ADD) v = __fadd_rn(v, __ldcg(a.resid + idx));
                    a.y[idx] = v;
                }
            }
        } else {
            __shared__ unsigned int s_last;
            float* part = a.partial + (static_cast<size_t>(blockIdx.z) * gridDim.y + blockIdx.y) * a.rows_padded;
            if (threadIdx.x < WT * 16) {
                const int wtl = threadIdx.x >> 4, r = threadIdx.x & 15;
                const int row = (base + wtl) * 16 + r;
                float v = 0.f;
#pragma unroll
                for (int k = 0; k < WK; ++k) v += rb[(wtl * WK + k) * 16 + r];
                if (row < a.rows_padded) __stcg(part + row, finite ? v * unscale : NAN);
            }
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) {
                unsigned int* ctr = a.counters + blockIdx.y * ((n_tiles + WT - 1) / WT) + base / WT;
                const unsigned int old = atomicAdd(ctr, 1u);
                s_last = (old == static_cast<unsigned int>(KS - 1));
                if (s_last) *ctr = 0u;                      // ready for the next launch
            }
            __syncthreads();
            if (s_last) {
                __threadfence();
                if (threadIdx.x < WT * 16) {
                    const int row = base * 16 + threadIdx.x;
                    if (row < q.rows) {
                        float v = 0.f;
                        for (int z = 0; z < KS; ++z)
                            v += __ldcg(a.partial + (static_cast<size_t>(z) * gridDim.y + blockIdx.y) * a.rows_padded + row);
                        const long long idx = (a.fused ? static_cast<long long>(blockIdx.y) * a.ldy : 0) + row;
                        if (a.epilogue == RWKVQ_EPI_RELU2) { v = fmaxf(v, 0.f); v = v * v; }
                        else if (a.epilogue == RWKVQ_EPI_ADD) v = __fadd_rn(v, __ldcg(a.resid + idx));
                        a.y[idx] = v;
                    }
                }
            }
        }
    }
}

// ------------------------------------------------------------ relayout kernels
__global__ void relayout_meta_kernel(QView t, uint32_t* out) {
    const int nsb = t.cols >> 8;
    const size_t total = static_cast<size_t>(t.rows) * nsb;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint8_t* mp = t.qsqm + i * 12;
        uint64_t qs = 0, qm = 0;
        for (int k = 0; k < 6; ++k) { qs |= static_cast<uint64_t>(mp[k]) << (8 * k); qm |= static_cast<uint64_t>(mp[6 + k]) << (8 * k); }
        const uint32_t dd = reinterpret_cast<const uint16_t*>(t.d)[i] |
                            (static_cast<uint32_t>(reinterpret_cast<const uint16_t*>(t.dm)[i]) << 16);
        for (int w = 0; w < 4; ++w)
            out[i * 4 + w] = sixbit(qs, 2 * w) | (sixbit(qs, 2 * w + 1) << 6) | (sixbit(qm, 2 * w) << 12) |
                             (sixbit(qm, 2 * w + 1) << 18) | (((dd >> (8 * w)) & 0xFFu) << 24);
    }
}

// One output word per thread.  `mode` 5: sb6@5, 6: sb6@6 (two words per block), 16: sym@6.
__global__ void relayout_planes_kernel(QView t, uint32_t* out, int mode) {
    const size_t words_per_row = mode == 5 ? (t.cols >> 5) : (t.cols >> 4);
    const size_t total = static_cast<size_t>(t.rows) * words_per_row;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t r = i / words_per_row, wi = i % words_per_row;
        const uint8_t* qh = t.qh + r * (t.cols >> 3);
        const uint8_t* qh2 = t.qh2 ? t.qh2 + r * (t.cols >> 3) : nullptr;
        uint32_t w = 0;
        if (mode == 5) {
            const int c0 = static_cast<int>(wi) * 32;
            for (int G = 0; G < 8; ++G)
                for (int b = 0; b < 4; ++b) {
                    const int wt = G < 4 ? 4 * G + b : 16 + 4 * (G - 4) + b;
                    w |= plane_bit(qh, c0 + wt) << (8 * b + G);
                }
        } else if (mode == 6) {
            const int c0 = static_cast<int>(wi >> 1) * 32, second = static_cast<int>(wi & 1);
            for (int j = 0; j < 4; ++j)
                for (int b = 0; b < 4; ++b) {
                    const int wt = second * 16 + 4 * j + b;
                    w |= plane_bit(qh, c0 + wt) << (8 * b + 2 * j);
                    w |= plane_bit(qh2, c0 + wt) << (8 * b + 2 * j + 1);
                }
        } else {
            const int c0 = static_cast<int>(wi) * 16;
            for (int G = 0; G < 4; ++G)
                for (int b = 0; b < 4; ++b) {
                    const int wt = G < 2 ? 4 * G + b : 8 + 4 * (G - 2) + b;
                    w |= plane_bit(qh, c0 + wt) << (8 * b + 2 * G);
                    w |= plane_bit(qh2, c0 + wt) << (8 * b + 2 * G + 1);
                }
        }
        out[i] = w;
    }
}

int mma_layout_of(const rwkvq_qtensor& t) {
    if (t.kind == RWKVQ_KIND_SB6 && t.dev_meta && (t.bits == 4 || t.dev_planes)) return ML_SB6_4 + (t.bits - 4);
    if (t.kind == RWKVQ_KIND_SYM && t.bits == 8) return ML_SYM8;
    if (t.kind == RWKVQ_KIND_SYM && t.bits == 6 && t.dev_planes) return ML_SYM6;
    return -1;
}

constexpr int kResidentCtas = 2 * 148;     // 2 CTAs of 256 threads per SM at <= 128 registers
constexpr int kSplitMaxRows = 4096;        // rows a K-split launch may have (scratch sizing)
constexpr int kSplitMaxSlices = 4;

// Scratch of a K-split launch: partial sums, then the (self-resetting) arrival counters.
size_t gemv_mma_scratch_bytes() {
    return sizeof(float) * kSplitMaxSlices * kMmaMaxFused * kSplitMaxRows + sizeof(unsigned int) * 1024;
}

template <int L, int WK>
static int launch_one(MmaArgs& a, int rows, int cols, int n_mats, int KS, cudaStream_t s) {
    constexpr int WT = kMmaWarps / WK;
    const size_t smem = 3 * static_cast<size_t>(cols) + 4 * (cols / 16) + 2 * kMmaWarps * 16 * 4;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<L, WK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
        if (e != cudaSuccess) return fail(RWKVQ_E_LIMIT, "gemv_mma: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    const int units = ((rows + 15) / 16 + WT - 1) / WT;
    const int cap = kResidentCtas / (n_mats * KS) > 0 ? kResidentCtas / (n_mats * KS) : 1;
    a.rows_padded = ((rows + 15) / 16) * 16;
    cudaError_t le = launch_pdl(gemv_mma_kernel<L, WK>, dim3(units < cap ? units : cap, n_mats, KS),
                                dim3(kMmaWarps * 32), smem, s, a);
    if (le != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "gemv_mma: %s", cudaGetErrorString(le));
    return RWKVQ_OK;
}

// Work split: a single wave of co-resident CTAs whenever the matrix allows it.
//   * few row tiles, long rows  -> K is also split across CTAs (needs scratch)
//   * tiles * n_mats <= resident CTAs -> one tile per CTA, its 8 warps split K
//   * more tiles -> WT tiles per CTA so that the grid still fits one wave
//   * very many tiles (head) -> persistent CTAs, 8 warps split K of each tile
template <int L>
static int launch_wk(MmaArgs& a, int rows, int cols, int n_mats, float* scratch, cudaStream_t s) {
    const int n_iters = cols / Geo<L>::KI;
    const int tiles = (rows + 15) / 16;
    int KS = 1;
    if (scratch && n_iters >= 16 && rows <= kSplitMaxRows) {
        if (tiles * n_mats * 4 <= kResidentCtas && n_iters >= 32) KS = 4;
        else if (tiles * n_mats * 2 <= kResidentCtas) KS = 2;
    }
    if (KS > 1) {
        a.partial = scratch;
        a.counters = reinterpret_cast<unsigned int*>(scratch + kSplitMaxSlices * kMmaMaxFused * kSplitMaxRows);
        return launch_one<L, 8>(a, rows, cols, n_mats, KS, s);
    }
    int wt = 1;
    if (tiles * n_mats > kResidentCtas) {
        wt = 0;
        for (int c = 2; c <= 8; c <<= 1)
            if (((tiles + c - 1) / c) * n_mats <= kResidentCtas && 8 / c <= n_iters) { wt = c; break; }
        if (wt == 0) wt = 1;                 // persistent loop
    }
    int wk = 8 / wt;
    while (wk > n_iters) wk >>= 1;           // short rows: fewer K slices, more tiles per CTA
    switch (wk) {
        case 8: return launch_one<L, 8>(a, rows, cols, n_mats, 1, s);
        case 4: return launch_one<L, 4>(a, rows, cols, n_mats, 1, s);
        case 2: return launch_one<L, 2>(a, rows, cols, n_mats, 1, s);
        default: return launch_one<L, 1>(a, rows, cols, n_mats, 1, s);
    }
}

// Launch the single-vector tensor-core GEMV for `n_mats` same-shape matrices.
// `scratch` (gemv_mma_scratch_bytes(), zero-initialised once, reusable) enables the
// K split across CTAs; nullptr disables it.
int launch_gemv_mma(int layout, const rwkvq_qtensor* ts, int n_mats, const void* x, int x_dtype,
                    long long ldx, float* y, long long ldy, int epilogue, const float* resid,
                    int fused, cudaStream_t s, const void* const* x_each, float* scratch) {
    MmaArgs a{};
    for (int k = 0; k < n_mats; ++k) { a.t[k] = make_view(ts[k]); a.xk[k] = x_each ? x_each[k] : nullptr; }
    a.x = x; a.x_dtype = x_dtype; a.ldx = ldx; a.y = y; a.ldy = ldy;
    a.resid = resid; a.epilogue = epilogue; a.fused = fused;
    const int rows = ts[0].rows, cols = ts[0].cols;
    switch (layout) {
        case ML_SB6_4: return launch_wk<ML_SB6_4>(a, rows, cols, n_mats, scratch, s);
        case ML_SB6_5: return launch_wk<ML_SB6_5>(a, rows, cols, n_mats, scratch, s);
        case ML_SB6_6: return launch_wk<ML_SB6_6>(a, rows, cols, n_mats, scratch, s);
        case ML_SYM6: return launch_wk<ML_SYM6>(a, rows, cols, n_mats, scratch, s);
        default: return launch_wk<ML_SYM8>(a, rows, cols, n_mats, scratch, s);
    }
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

int rwkvq_relayout_meta(const rwkvq_qtensor* t, void* meta_out, void* stream) {
    int rc = validate_qtensor(t, "rwkvq_relayout_meta");
    if (rc) return rc;
    RWKVQ_REQUIRE(t->kind == RWKVQ_KIND_SB6, RWKVQ_E_DTYPE, "rwkvq_relayout_meta: only sb6 tensors have scale records");
    RWKVQ_REQUIRE(meta_out != nullptr && aligned(meta_out, 16), RWKVQ_E_ALIGN, "rwkvq_relayout_meta: out must be 16-byte aligned");
    relayout_meta_kernel<<<148 * 4, 256, 0, static_cast<cudaStream_t>(stream)>>>(make_view(*t),
                                                                                 static_cast<uint32_t*>(meta_out));
    return check_launch("rwkvq_relayout_meta");
}

int rwkvq_relayout_planes(const rwkvq_qtensor* t, void* planes_out, void* stream) {
    int rc = validate_qtensor(t, "rwkvq_relayout_planes");
    if (rc) return rc;
    int mode = 0;
    if (t->kind == RWKVQ_KIND_SB6 && t->bits == 5) mode = 5;
    else if (t->kind == RWKVQ_KIND_SB6 && t->bits == 6) mode = 6;
    else if (t->kind == RWKVQ_KIND_SYM && t->bits == 6) mode = 16;
    RWKVQ_REQUIRE(mode != 0, RWKVQ_E_DTYPE, "rwkvq_relayout_planes: tensor has no bit-planes");
    RWKVQ_REQUIRE(planes_out != nullptr && aligned(planes_out, 16), RWKVQ_E_ALIGN,
                  "rwkvq_relayout_planes: out must be 16-byte aligned");
    relayout_planes_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        make_view(*t), static_cast<uint32_t*>(planes_out), mode);
    return check_launch("rwkvq_relayout_planes");
}

}  // extern "C"

// ------------------------------------------------- K-split GEMV, built-in scratch
// The K-split launch needs room for the slices' partial row sums and for its
// arrival counters.  This variant keeps that room in the module image, so the call
// path never asks the CUDA allocator for anything.
namespace rwkvq {

constexpr int kStaticMaxRows = kSplitMaxRows;     // largest OUT served
constexpr int kStaticMaxCols = 16384;             // largest IN served (shared-memory staging of x)
constexpr size_t kStaticPartialFloats = static_cast<size_t>(kSplitMaxSlices) * kMmaMaxFused * kSplitMaxRows;
constexpr size_t kStaticCounterWords = 1024;
constexpr int kStaticMaxDevices = 64;

// 256 KiB of partial sums followed by 4 KiB of counters; zero at module load.
static __device__ __align__(256) float g_static_scratch[kStaticPartialFloats + kStaticCounterWords];

// Device address of the scratch on the current device, looked up once per device.
static int static_scratch(float** out) {
    static float* ptrs[kStaticMaxDevices] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_gemv_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kStaticMaxDevices)
        return fail(RWKVQ_E_LIMIT, "rwkvq_gemv_static: device ordinal %d, at most %d devices", dev, kStaticMaxDevices);
    float* p = __atomic_load_n(&ptrs[dev], __ATOMIC_ACQUIRE);
    if (p == nullptr) {
        void* sym = nullptr;
        e = cudaGetSymbolAddress(&sym, g_static_scratch);
        if (e != cudaSuccess || sym == nullptr)
            return fail(RWKVQ_E_LAUNCH, "rwkvq_gemv_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        p = static_cast<float*>(sym);
        __atomic_store_n(&ptrs[dev], p, __ATOMIC_RELEASE);   // racing threads store the same address
    }
    *out = p;
    return RWKVQ_OK;
}

}  // namespace rwkvq

extern "C" int rwkvq_gemv_static(const rwkvq_qtensor* t, const void* x, int x_dtype, float* y, int epilogue,
                                 const float* resid, void* stream) {
    int rc = validate_qtensor(t, "rwkvq_gemv_static");
    if (rc) return rc;
    RWKVQ_REQUIRE(x != nullptr && y != nullptr, RWKVQ_E_NULL, "rwkvq_gemv_static: x or y is null");
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F32 || x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_DTYPE,
                  "rwkvq_gemv_static: x_dtype %d", x_dtype);
    RWKVQ_REQUIRE(aligned(x, 16), RWKVQ_E_ALIGN, "rwkvq_gemv_static: x must be 16-byte aligned");
    RWKVQ_REQUIRE(epilogue >= RWKVQ_EPI_NONE && epilogue <= RWKVQ_EPI_ADD, RWKVQ_E_DTYPE,
                  "rwkvq_gemv_static: epilogue %d", epilogue);
    RWKVQ_REQUIRE(epilogue != RWKVQ_EPI_ADD || resid != nullptr, RWKVQ_E_NULL, "rwkvq_gemv_static: resid is null");
    const int ml = mma_layout_of(*t);
    RWKVQ_REQUIRE(ml >= 0, RWKVQ_E_DTYPE,
                  "rwkvq_gemv_static: needs an sb6 tensor with relayouted records/planes or a sym tensor");
    RWKVQ_REQUIRE(t->rows <= kStaticMaxRows && t->cols <= kStaticMaxCols, RWKVQ_E_LIMIT,
                  "rwkvq_gemv_static: [%d, %d] exceeds the built-in scratch, at most [%d, %d]", t->rows, t->cols,
                  kStaticMaxRows, kStaticMaxCols);
    float* scratch = nullptr;
    rc = static_scratch(&scratch);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the arrival counters must read zero when the kernel starts
    cudaError_t e = cudaMemsetAsync(scratch + kStaticPartialFloats, 0, kStaticCounterWords * sizeof(unsigned int), s);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_gemv_static: cudaMemsetAsync: %s", cudaGetErrorString(e));
    rc = launch_gemv_mma(ml, t, 1, x, x_dtype, t->cols, y, t->rows, epilogue, resid, 0, s, nullptr, scratch);
    return rc ? rc : check_launch("rwkvq_gemv_static");
}
