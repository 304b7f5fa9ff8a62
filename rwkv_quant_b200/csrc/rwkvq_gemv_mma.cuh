// Device-side building blocks of the integer tensor-core GEMV.
//
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
#pragma once
#include "rwkvq_common.cuh"

namespace rwkvq {

enum MmaLayout { ML_SB6_4 = 0, ML_SB6_5, ML_SB6_6, ML_SYM6, ML_SYM8, ML_RTN8 };   // RTN8: int8 codes, one fp16 scale per row

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
template <> struct Geo<ML_RTN8> { static constexpr int KI = 128, BLK = 16, BITS = 8; };

// Fixed-point bits of the activation: |sum over one block of q*X| must stay below 2^31.
template <int L> __host__ __device__ constexpr int x_bits() { return (L == ML_SYM8 || L == ML_RTN8) ? 19 : 20; }

// Everything thread (g, t) streams for one iteration (8 blocks) of rows g, g+8.
struct FragData {
    uint4 ca[2], cb[2];    // codes of blocks 2t, 2t+1: row g (ca), row g+8 (cb)
    uint4 ma, mb;          // sb6: 16-byte scale records;  sym: .x,.y = 8 scale codes, .z = d bits
    uint4 pa, pb;          // regrouped bit-planes of the two blocks
};
template <int L>
using Frag = FragData;     // the same registers for every layout; L selects how they are filled

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
// zflag (optional, sb6 and 6-bit sym): per aligned group of 32 columns, 1 = the activations of
// the group are all zero (prepare_x); the 16 bytes of codes of such a group are not read and the
// fragment keeps whatever it held, which the zero activations multiply.
template <int L>
__device__ __forceinline__ void load_frag(Frag<L>& f, const QView& q, int r0, int r1, int it, int t,
                                          const uint8_t* zflag = nullptr) {
    const size_t R0 = static_cast<size_t>(r0), R1 = static_cast<size_t>(r1);
    if (L <= ML_SB6_6) {
        const int nsb = q.cols >> 8;
        const size_t rowb = static_cast<size_t>(q.cols >> 1), nb = static_cast<size_t>(q.cols >> 5);
        const uint8_t* p0 = q.codes + R0 * rowb + it * 128 + t * 32;
        const uint8_t* p1 = q.codes + R1 * rowb + it * 128 + t * 32;
        const bool z0 = zflag != nullptr && zflag[it * 8 + 2 * t] != 0, z1 = zflag != nullptr && zflag[it * 8 + 2 * t + 1] != 0;
        if (!z0) { f.ca[0] = ld_stream_u128(p0); f.cb[0] = ld_stream_u128(p1); }
        if (!z1) { f.ca[1] = ld_stream_u128(p0 + 16); f.cb[1] = ld_stream_u128(p1 + 16); }
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
            if (zflag == nullptr || zflag[it * 4 + t] == 0) {
                f.ca[0] = ld_stream_u128(q.codes + R0 * rowb + it * 64 + t * 16);
                f.cb[0] = ld_stream_u128(q.codes + R1 * rowb + it * 64 + t * 16);
            }
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
        if (L == ML_RTN8) {             // one scale per row
            f.ma = make_uint4(0, 0, ld_stream_u16(static_cast<const __half*>(q.scale) + R0), 0);
            f.mb = make_uint4(0, 0, ld_stream_u16(static_cast<const __half*>(q.scale) + R1), 0);
        } else {
            const uint2 sa = ld_stream_u64(reinterpret_cast<const uint8_t*>(q.qs) + R0 * nb16 + it * 8);
            const uint2 sb = ld_stream_u64(reinterpret_cast<const uint8_t*>(q.qs) + R1 * nb16 + it * 8);
            f.ma = make_uint4(sa.x, sa.y, ld_stream_u16(q.d + R0 * nsb + (it >> 1)), 0);
            f.mb = make_uint4(sb.x, sb.y, ld_stream_u16(q.d + R1 * nsb + (it >> 1)), 0);
        }
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
// zflag (optional): zflag[c / 32] = 1 where all 32 fixed-point activations of the aligned group are zero: the
// weights of such a group contribute exactly nothing (integer products, and the block min
// multiplies the group's sum), so the loader may leave them unread (load_frag).
__device__ __forceinline__ float prepare_x(const void* x, int dtype, int n_in, int bits, int8_t* dig,
                                           float* xs16, float* red, bool& finite, uint8_t* zflag) {
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
        // 8 consecutive lanes cover 32 columns (whole warps get here together)
        if (zflag != nullptr) {
            const unsigned nz = __ballot_sync(0xFFFFFFFFu, (X0 | X1 | X2 | X3) != 0);
            if ((tid & 7) == 0) zflag[i >> 3] = ((nz >> (tid & 24)) & 0xFFu) == 0u;
        }
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

// Consume one fragment: the 2 x 2 (row, block) dot products of this thread for
// iteration `it` (index of the group of 8 blocks inside the prepared activations),
// scaled and added to the accumulators of rows g (acc0) and g + 8 (acc1).
// Which B columns a lane feeds: column 2t+dg of MMA set 1, column 2t of set 2.
template <int L>
__device__ __forceinline__ void consume_frag(const Frag<L>& cur, int it, int g, int t, const int8_t* dig, int n_in,
                                             const float* xs16, float& acc0, float& acc1) {
    constexpr bool SB6 = L <= ML_SB6_6;
    constexpr bool A_UNSIGNED = L != ML_SYM8 && L != ML_RTN8;
    const bool b_set1 = (g >> 1) == t;
    const bool b_set2 = g == 2 * t;
    const int8_t* dig1 = dig + (g & 1) * n_in;
    const int8_t* dig3 = dig + 2 * n_in;
    float2 sa, sb, ma = make_float2(0.f, 0.f), mb = ma;
    if (SB6) {
        sb6_pair_scales(cur.ma, t, sa, ma);
        sb6_pair_scales(cur.mb, t, sb, mb);
    } else if (L == ML_RTN8) {
        const float s0 = __half2float(__ushort_as_half(static_cast<unsigned short>(cur.ma.z)));
        const float s1 = __half2float(__ushort_as_half(static_cast<unsigned short>(cur.mb.z)));
        sa = make_float2(s0, s0);
        sb = make_float2(s1, s1);
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

}  // namespace rwkvq
