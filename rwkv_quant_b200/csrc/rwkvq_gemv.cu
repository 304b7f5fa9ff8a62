// Decode GEMV family: y[n, o] = epi(sum_c W[o, c] x[n, c]) with W streamed in
// the .rwkvq file layout (sb6 int4/5/6, sym 6/8, per-row int8) and never
// materialised.
//
// Work split: a warp owns R output rows; lane l owns the 32-column chunks
// p = l, l+32, ... of those rows, so one warp-wide load instruction reads 512
// contiguous bytes of nibble codes per row.  The activation chunk lives in
// registers (pre-scaled by 2^64) and is reused for the R rows.  Codes enter the
// FFMA as subnormal floats (see byte_as_subnormal), so unpacking costs one PRMT
// per weight and no int->float conversion.  fp32 accumulation, warp-shuffle
// reduction at the end.
#include "rwkvq_common.cuh"

namespace rwkvq {

enum ChunkKind { CK_SB6_4 = 0, CK_SB6_5, CK_SB6_6, CK_SYM6, CK_SYM8, CK_RTN8 };

constexpr int kWarpsPerCta = 4;
constexpr int kMaxFused = 4;

struct GemvArgs {
    QView t[kMaxFused];   // t[blockIdx.y]
    const void* x;        // [n_mats or N, ldx]
    int x_dtype;
    long long ldx;
    float* y;
    long long ldy;
    const float* resid;
    int epilogue;
    int n_cols;           // right-hand sides handled by this launch (<= NC)
    int fused;            // 1: blockIdx.y selects matrix AND input row; output row stride ldy
};

__device__ __forceinline__ float apply_epilogue(float v, int epi, const float* resid, long long idx) {
    if (epi == RWKVQ_EPI_RELU2) {
        v = fmaxf(v, 0.0f);
        return v * v;
    }
    if (epi == RWKVQ_EPI_ADD) return __fadd_rn(v, __ldcg(resid + idx));
    return v;
}

// 32 activations of chunk p, scaled by 2^64, plus their plain sums per 16.
__device__ __forceinline__ void load_x_chunk(const void* x, int dtype, int p, float (&xs)[32],
                                             float& sum_lo, float& sum_hi) {
    if (dtype == RWKVQ_F32) {
        const float4* xp = reinterpret_cast<const float4*>(static_cast<const float*>(x) + p * 32);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 v = __ldcg(xp + i);
            xs[4 * i + 0] = v.x; xs[4 * i + 1] = v.y; xs[4 * i + 2] = v.z; xs[4 * i + 3] = v.w;
        }
    } else {
        const uint4* xp = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + p * 32);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 v = __ldcg(xp + i);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float a, b;
                if (dtype == RWKVQ_F16) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
                    a = f.x; b = f.y;
                } else {
                    a = __uint_as_float(w[k] << 16);
                    b = __uint_as_float(w[k] & 0xFFFF0000u);
                }
                xs[8 * i + 2 * k] = a; xs[8 * i + 2 * k + 1] = b;
            }
        }
    }
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) { s0 += xs[i]; s1 += xs[16 + i]; }
    sum_lo = s0; sum_hi = s1;
#pragma unroll
    for (int i = 0; i < 32; ++i) xs[i] *= kXPreScale;
}

// dot of the 4 bytes of `w` (as subnormal floats) with xs[base .. base+3]
template <int NC>
__device__ __forceinline__ void dot4(uint32_t w, const float (&xs)[NC][32], int base, float (&dv)[NC]) {
    const float f0 = byte_as_subnormal<0>(w), f1 = byte_as_subnormal<1>(w);
    const float f2 = byte_as_subnormal<2>(w), f3 = byte_as_subnormal<3>(w);
#pragma unroll
    for (int n = 0; n < NC; ++n) {
        dv[n] = fmaf(xs[n][base + 0], f0, dv[n]);
        dv[n] = fmaf(xs[n][base + 1], f1, dv[n]);
        dv[n] = fmaf(xs[n][base + 2], f2, dv[n]);
        dv[n] = fmaf(xs[n][base + 3], f3, dv[n]);
    }
}

template <int KIND>
struct Chunk;

// ---- sb6: 16 B nibbles (+4 B per bit-plane) + 12 B / super-block of scale codes
template <int BITS>
struct ChunkSb6 {
    uint4 c;
    uint32_t h, h2, m0, m1, m2, dd, ddm;
    __device__ __forceinline__ void load(const QView& t, int row, int p) {
        const size_t R = static_cast<size_t>(row);
        const int nsb = t.cols >> 8, sbi = p >> 3;
        c = ld_stream_u128(t.codes + R * (t.cols >> 1) + p * 16);
        h = h2 = 0;
        if (BITS >= 5) h = ld_stream_u32(t.qh + R * (t.cols >> 3) + p * 4);
        if (BITS >= 6) h2 = ld_stream_u32(t.qh2 + R * (t.cols >> 3) + p * 4);
        const uint8_t* mp = t.qsqm + (R * nsb + sbi) * 12;
        m0 = ld_stream_u32(mp); m1 = ld_stream_u32(mp + 4); m2 = ld_stream_u32(mp + 8);
        dd = ld_stream_u16(t.d + R * nsb + sbi);
        ddm = ld_stream_u16(t.dm + R * nsb + sbi);
    }
    template <int NC>
    __device__ __forceinline__ void accumulate(int p, const float (&xs)[NC][32],
                                               const float (&s_lo)[NC], const float (&s_hi)[NC],
                                               float (&acc)[NC]) const {
        float s, m;
        sb6_scale_min(m0, m1, m2, p & 7, half_bits_to_float(dd), half_bits_to_float(ddm), s, m);
        float dv[NC];
#pragma unroll
        for (int n = 0; n < NC; ++n) dv[n] = 0.f;
        const uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t lo = w[i] & 0x0F0F0F0Fu, hi = (w[i] >> 4) & 0x0F0F0F0Fu;
            if (BITS >= 5) {
                lo |= spread_nibble<4>((h >> (4 * i)) & 0xFu);
                hi |= spread_nibble<4>((h >> (16 + 4 * i)) & 0xFu);
            }
            if (BITS >= 6) {
                lo |= spread_nibble<5>((h2 >> (4 * i)) & 0xFu);
                hi |= spread_nibble<5>((h2 >> (16 + 4 * i)) & 0xFu);
            }
            dot4<NC>(lo, xs, 4 * i, dv);
            dot4<NC>(hi, xs, 16 + 4 * i, dv);
        }
        const float ss = s * kCodeUnscale;
#pragma unroll
        for (int n = 0; n < NC; ++n) acc[n] = fmaf(ss, dv[n], fmaf(m, s_lo[n] + s_hi[n], acc[n]));
    }
};
template <> struct Chunk<CK_SB6_4> : ChunkSb6<4> {};
template <> struct Chunk<CK_SB6_5> : ChunkSb6<5> {};
template <> struct Chunk<CK_SB6_6> : ChunkSb6<6> {};

// ---- sym@6: two blocks of 16, codes stored +32 as nibble + two bit-planes
template <>
struct Chunk<CK_SYM6> {
    uint4 c;
    uint32_t h, h2, qs2, dd;
    __device__ __forceinline__ void load(const QView& t, int row, int p) {
        const size_t R = static_cast<size_t>(row);
        c = ld_stream_u128(t.codes + R * (t.cols >> 1) + p * 16);
        h = ld_stream_u32(t.qh + R * (t.cols >> 3) + p * 4);
        h2 = ld_stream_u32(t.qh2 + R * (t.cols >> 3) + p * 4);
        qs2 = ld_stream_u16(t.qs + R * (t.cols >> 4) + p * 2);
        dd = ld_stream_u16(t.d + R * (t.cols >> 8) + (p >> 3));
    }
    template <int NC>
    __device__ __forceinline__ void accumulate(int, const float (&xs)[NC][32],
                                               const float (&s_lo)[NC], const float (&s_hi)[NC],
                                               float (&acc)[NC]) const {
        const float d = half_bits_to_float(dd);
        const uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const int qs = static_cast<int8_t>((qs2 >> (8 * b)) & 0xFFu);
            const float s = half_roundtrip(__fmul_rn(static_cast<float>(qs), d));
            float dv[NC];
#pragma unroll
            for (int n = 0; n < NC; ++n) dv[n] = 0.f;
#pragma unroll
            for (int i = 0; i < 2; ++i) {       // word i of the block: bytes 4i..4i+3
                const uint32_t ww = w[2 * b + i];
                const int c_lo = 16 * b + 4 * i, c_hi = c_lo + 8;
                uint32_t lo = ww & 0x0F0F0F0Fu, hi = (ww >> 4) & 0x0F0F0F0Fu;
                lo |= spread_nibble<4>((h >> c_lo) & 0xFu) | spread_nibble<5>((h2 >> c_lo) & 0xFu);
                hi |= spread_nibble<4>((h >> c_hi) & 0xFu) | spread_nibble<5>((h2 >> c_hi) & 0xFu);
                dot4<NC>(lo, xs, c_lo, dv);
                dot4<NC>(hi, xs, c_hi, dv);
            }
            const float ss = s * kCodeUnscale, sb = -32.f * s;
#pragma unroll
            for (int n = 0; n < NC; ++n)
                acc[n] = fmaf(ss, dv[n], fmaf(sb, b ? s_hi[n] : s_lo[n], acc[n]));
        }
    }
};

// ---- sym@8: two blocks of 16 signed bytes
template <>
struct Chunk<CK_SYM8> {
    uint4 c0, c1;
    uint32_t qs2, dd;
    __device__ __forceinline__ void load(const QView& t, int row, int p) {
        const size_t R = static_cast<size_t>(row);
        const uint8_t* cp = t.codes + R * t.cols + p * 32;
        c0 = ld_stream_u128(cp); c1 = ld_stream_u128(cp + 16);
        qs2 = ld_stream_u16(t.qs + R * (t.cols >> 4) + p * 2);
        dd = ld_stream_u16(t.d + R * (t.cols >> 8) + (p >> 3));
    }
    template <int NC>
    __device__ __forceinline__ void accumulate(int, const float (&xs)[NC][32],
                                               const float (&s_lo)[NC], const float (&s_hi)[NC],
                                               float (&acc)[NC]) const {
        const float d = half_bits_to_float(dd);
        const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const int qs = static_cast<int8_t>((qs2 >> (8 * b)) & 0xFFu);
            const float s = half_roundtrip(__fmul_rn(static_cast<float>(qs), d));
            float dv[NC];
#pragma unroll
            for (int n = 0; n < NC; ++n) dv[n] = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i)     // code + 128 as an unsigned byte
                dot4<NC>(w[4 * b + i] ^ 0x80808080u, xs, 16 * b + 4 * i, dv);
            const float ss = s * kCodeUnscale, sb = -128.f * s;
#pragma unroll
            for (int n = 0; n < NC; ++n)
                acc[n] = fmaf(ss, dv[n], fmaf(sb, b ? s_hi[n] : s_lo[n], acc[n]));
        }
    }
};

// ---- per-row int8: 32 signed bytes, the row scale is applied at the end
template <>
struct Chunk<CK_RTN8> {
    uint4 c0, c1;
    __device__ __forceinline__ void load(const QView& t, int row, int p) {
        const uint8_t* cp = t.codes + static_cast<size_t>(row) * t.cols + p * 32;
        c0 = ld_stream_u128(cp); c1 = ld_stream_u128(cp + 16);
    }
    template <int NC>
    __device__ __forceinline__ void accumulate(int, const float (&xs)[NC][32],
                                               const float (&s_lo)[NC], const float (&s_hi)[NC],
                                               float (&acc)[NC]) const {
        const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        float dv[NC];
#pragma unroll
        for (int n = 0; n < NC; ++n) dv[n] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) dot4<NC>(w[i] ^ 0x80808080u, xs, 4 * i, dv);
#pragma unroll
        for (int n = 0; n < NC; ++n)
            acc[n] = fmaf(kCodeUnscale, dv[n], fmaf(-128.f, s_lo[n] + s_hi[n], acc[n]));
    }
};

template <int KIND, int R, int NC>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
gemv_chunk_kernel(const GemvArgs a) {
    pdl_wait();
    const QView& t = a.t[blockIdx.y];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = (blockIdx.x * kWarpsPerCta + warp) * R;
    if (row0 >= t.rows) return;
    const int n_chunks = t.cols >> 5;
    const size_t esz = (a.x_dtype == RWKVQ_F32) ? 4 : 2;
    const char* xbase = static_cast<const char*>(a.x) + (a.fused ? blockIdx.y * a.ldx * esz : 0);

    float acc[R][NC];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int n = 0; n < NC; ++n) acc[r][n] = 0.f;

    for (int p = lane; p < n_chunks; p += 32) {
        Chunk<KIND> ch[R];
#pragma unroll
        for (int r = 0; r < R; ++r) ch[r].load(t, min(row0 + r, t.rows - 1), p);
        float xs[NC][32], s_lo[NC], s_hi[NC];
#pragma unroll
        for (int n = 0; n < NC; ++n) {
            const int col = (n < a.n_cols) ? n : 0;
            load_x_chunk(xbase + col * a.ldx * esz, a.x_dtype, p, xs[n], s_lo[n], s_hi[n]);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) ch[r].template accumulate<NC>(p, xs, s_lo, s_hi, acc[r]);
    }

#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int n = 0; n < NC; ++n) {
            float v = acc[r][n];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            acc[r][n] = v;
        }
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = row0 + r;
            if (row >= t.rows) break;
            float rs = 1.f;
            if (KIND == CK_RTN8) rs = __half2float(static_cast<const __half*>(t.scale)[row]);
#pragma unroll
            for (int n = 0; n < NC; ++n) {
                if (n >= a.n_cols) break;
                const long long idx = (a.fused ? blockIdx.y : n) * a.ldy + row;
                a.y[idx] = apply_epilogue(__fmul_rn(acc[r][n], rs), a.epilogue, a.resid, idx);
            }
        }
    }
}

// Any layout / ragged shape: a warp per row, lanes stride over columns and
// decode element by element.  Slow; serves dense bf16, rtn nibbles, asym in
// [out, in] orientation and shapes the chunk kernels reject.
__global__ void __launch_bounds__(kWarpsPerCta * 32) gemv_generic_kernel(const GemvArgs a) {
    pdl_wait();
    const QView& t = a.t[0];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * kWarpsPerCta + warp;
    if (row >= t.rows) return;
    for (int n = 0; n < a.n_cols; ++n) {
        float acc = 0.f;
        for (int c = lane; c < t.cols; c += 32) {
            float xv;
            if (a.x_dtype == RWKVQ_F32) xv = static_cast<const float*>(a.x)[n * a.ldx + c];
            else if (a.x_dtype == RWKVQ_F16) xv = __half2float(static_cast<const __half*>(a.x)[n * a.ldx + c]);
            else xv = __bfloat162float(static_cast<const __nv_bfloat16*>(a.x)[n * a.ldx + c]);
            acc = fmaf(decode_element(t, row, c), xv, acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
        if (lane == 0) {
            const long long idx = n * a.ldy + row;
            a.y[idx] = apply_epilogue(acc, a.epilogue, a.resid, idx);
        }
    }
}

static int chunk_kind_of(const rwkvq_qtensor& t) {
    if (t.kind == RWKVQ_KIND_SB6) return CK_SB6_4 + (t.bits - 4);
    if (t.kind == RWKVQ_KIND_SYM) return t.bits == 6 ? CK_SYM6 : CK_SYM8;
    if (t.kind == RWKVQ_KIND_RTN && t.bits > 4 && t.cols % 32 == 0 && aligned(t.codes, 16)) return CK_RTN8;
    return -1;
}

static int rows_per_warp(const rwkvq_qtensor& t, int n_mats) {
    const long long weights = static_cast<long long>(t.rows) * t.cols * n_mats;
    if (t.rows >= 32768) return 8;
    if (weights >= (1ll << 24)) return 4;
    return 2;
}

template <int KIND, int NC>
static void launch_chunk(const GemvArgs& a, int rows, int n_mats, int R, cudaStream_t s) {
    const dim3 block(kWarpsPerCta * 32);
    auto grid = [&](int r) { return dim3((rows + kWarpsPerCta * r - 1) / (kWarpsPerCta * r), n_mats); };
    if (NC > 1) {   // register budget: the activation chunks of NC columns live in registers
        gemv_chunk_kernel<KIND, 2, NC><<<grid(2), block, 0, s>>>(a);
        return;
    }
    switch (R) {
        case 8: gemv_chunk_kernel<KIND, 8, NC><<<grid(8), block, 0, s>>>(a); break;
        case 4: gemv_chunk_kernel<KIND, 4, NC><<<grid(4), block, 0, s>>>(a); break;
        default: gemv_chunk_kernel<KIND, 2, NC><<<grid(2), block, 0, s>>>(a); break;
    }
}

template <int NC>
static void dispatch_kind(int ck, const GemvArgs& a, int rows, int n_mats, int R, cudaStream_t s) {
    switch (ck) {
        case CK_SB6_4: launch_chunk<CK_SB6_4, NC>(a, rows, n_mats, R, s); break;
        case CK_SB6_5: launch_chunk<CK_SB6_5, NC>(a, rows, n_mats, R, s); break;
        case CK_SB6_6: launch_chunk<CK_SB6_6, NC>(a, rows, n_mats, R, s); break;
        case CK_SYM6: launch_chunk<CK_SYM6, NC>(a, rows, n_mats, R, s); break;
        case CK_SYM8: launch_chunk<CK_SYM8, NC>(a, rows, n_mats, R, s); break;
        default: launch_chunk<CK_RTN8, NC>(a, rows, n_mats, R, s); break;
    }
}

static int check_x(const void* x, int x_dtype, long long ldx, const char* who) {
    RWKVQ_REQUIRE(x != nullptr, RWKVQ_E_NULL, "%s: x is null", who);
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F32 || x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_DTYPE,
                  "%s: x_dtype %d", who, x_dtype);
    return RWKVQ_OK;
}

static int check_x_vector_loads(const void* x, int x_dtype, long long ldx, const char* who) {
    const size_t esz = x_dtype == RWKVQ_F32 ? 4 : 2;
    RWKVQ_REQUIRE(aligned(x, 16) && (ldx * esz) % 16 == 0, RWKVQ_E_ALIGN,
                  "%s: x and its row stride must be 16-byte aligned", who);
    return RWKVQ_OK;
}

}  // namespace rwkvq

using namespace rwkvq;

namespace rwkvq {
// Sparse outlier overrides of a per-row tensor (formats/codec.py:279-292: W[r, c] = value after the
// dequantisation; the Metal kernel's CSR tail, backends/metal/quant_linear_v2.py:47-55): the product over
// the packed codes is short of sum_j (value_j - quantized_j) x[n, c_j] for the overrides j of row r.
// One thread per (right-hand side, row) adds its row's terms in column order (deterministic) and
// applies the epilogue, which the product launch therefore leaves out.
__global__ void __launch_bounds__(256) outlier_tail_kernel(const int* __restrict__ row_ptr, const int* __restrict__ cols,
                                                           const float* __restrict__ delta, const void* __restrict__ x,
                                                           int x_dtype, long long ldx, float* __restrict__ y, long long ldy,
                                                           const float* __restrict__ resid, int epilogue, int rows, int N) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= static_cast<long long>(rows) * N) return;
    const int n = static_cast<int>(i / rows), r = static_cast<int>(i - static_cast<long long>(n) * rows);
    float v = y[n * ldy + r];
    for (int j = row_ptr[r]; j < row_ptr[r + 1]; ++j) {
        const long long xi = n * ldx + cols[j];
        const float xv = x_dtype == RWKVQ_F32 ? static_cast<const float*>(x)[xi]
                       : x_dtype == RWKVQ_F16 ? __half2float(static_cast<const __half*>(x)[xi])
                                              : __bfloat162float(static_cast<const __nv_bfloat16*>(x)[xi]);
        v = fmaf(xv, delta[j], v);
    }
    if (epilogue == RWKVQ_EPI_RELU2) { v = fmaxf(v, 0.f); v = v * v; }
    else if (epilogue == RWKVQ_EPI_ADD) v = __fadd_rn(v, resid[n * ldy + r]);
    y[n * ldy + r] = v;
}
}  // namespace rwkvq

extern "C" {

int rwkvq_gemv(const rwkvq_qtensor* t, const void* x, int x_dtype, int N, int64_t ldx, float* y,
               int64_t ldy, int epilogue, const float* resid, void* stream) {
    int rc = validate_qtensor(t, "rwkvq_gemv");
    if (rc) return rc;
    rc = check_x(x, x_dtype, ldx, "rwkvq_gemv");
    if (rc) return rc;
    RWKVQ_REQUIRE(y != nullptr, RWKVQ_E_NULL, "rwkvq_gemv: y is null");
    RWKVQ_REQUIRE(N >= 1, RWKVQ_E_SHAPE, "rwkvq_gemv: N=%d", N);
    RWKVQ_REQUIRE(ldx >= t->cols && ldy >= t->rows, RWKVQ_E_SHAPE, "rwkvq_gemv: ldx=%lld ldy=%lld too small",
                  (long long)ldx, (long long)ldy);
    RWKVQ_REQUIRE(epilogue >= RWKVQ_EPI_NONE && epilogue <= RWKVQ_EPI_ADD, RWKVQ_E_DTYPE,
                  "rwkvq_gemv: epilogue %d", epilogue);
    RWKVQ_REQUIRE(epilogue != RWKVQ_EPI_ADD || resid != nullptr, RWKVQ_E_NULL, "rwkvq_gemv: resid is null");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    GemvArgs a{};
    a.t[0] = make_view(*t);
    a.x_dtype = x_dtype; a.ldx = ldx; a.ldy = ldy; a.epilogue = epilogue; a.fused = 0;
    const int ck = chunk_kind_of(*t);
    const size_t esz = x_dtype == RWKVQ_F32 ? 4 : 2;
    if (ck < 0) {
        a.x = x; a.y = y; a.resid = resid; a.n_cols = N;
        gemv_generic_kernel<<<(t->rows + kWarpsPerCta - 1) / kWarpsPerCta, kWarpsPerCta * 32, 0, s>>>(a);
        return check_launch("rwkvq_gemv(generic)");
    }
    rc = check_x_vector_loads(x, x_dtype, ldx, "rwkvq_gemv");
    if (rc) return rc;
    const int ml = mma_layout_of(*t);
    if (ml >= 0) {      // one launch per right-hand side: each column's result is independent of N
        for (int n = 0; n < N; ++n) {
            rc = launch_gemv_mma(ml, t, 1, static_cast<const char*>(x) + static_cast<size_t>(n) * ldx * esz, x_dtype,
                                 ldx, y + static_cast<size_t>(n) * ldy, ldy, epilogue,
                                 resid ? resid + static_cast<size_t>(n) * ldy : nullptr, 0, s);
            if (rc) return rc;
        }
        return check_launch("rwkvq_gemv(mma)");
    }
    const int R = rows_per_warp(*t, 1);
    for (int n0 = 0; n0 < N;) {
        const int left = N - n0;
        a.x = static_cast<const char*>(x) + static_cast<size_t>(n0) * ldx * esz;
        a.y = y + static_cast<size_t>(n0) * ldy;
        a.resid = resid ? resid + static_cast<size_t>(n0) * ldy : nullptr;
        if (left >= 2) {
            a.n_cols = 2;
            dispatch_kind<2>(ck, a, t->rows, 1, R, s);
            n0 += 2;
        } else {
            a.n_cols = 1;
            dispatch_kind<1>(ck, a, t->rows, 1, R, s);
            n0 += 1;
        }
    }
    return check_launch("rwkvq_gemv");
}

int rwkvq_gemv_fused(const rwkvq_qtensor* ts, int K, const void* x, int x_dtype, float* y,
                     void* stream) {
    RWKVQ_REQUIRE(ts != nullptr, RWKVQ_E_NULL, "rwkvq_gemv_fused: tensor array is null");
    RWKVQ_REQUIRE(K >= 1 && K <= kMaxFused, RWKVQ_E_LIMIT, "rwkvq_gemv_fused: K=%d, at most %d", K, kMaxFused);
    for (int k = 0; k < K; ++k) {
        int rc = validate_qtensor(ts + k, "rwkvq_gemv_fused");
        if (rc) return rc;
        RWKVQ_REQUIRE(ts[k].kind == ts[0].kind && ts[k].bits == ts[0].bits && ts[k].rows == ts[0].rows &&
                          ts[k].cols == ts[0].cols,
                      RWKVQ_E_SHAPE, "rwkvq_gemv_fused: matrix %d differs in layout or shape", k);
    }
    int rc = check_x(x, x_dtype, ts[0].cols, "rwkvq_gemv_fused");
    if (rc) return rc;
    rc = check_x_vector_loads(x, x_dtype, ts[0].cols, "rwkvq_gemv_fused");
    if (rc) return rc;
    RWKVQ_REQUIRE(y != nullptr, RWKVQ_E_NULL, "rwkvq_gemv_fused: y is null");
    int ml = mma_layout_of(ts[0]);
    for (int k = 1; k < K; ++k)
        if (mma_layout_of(ts[k]) != ml) ml = -1;
    if (ml >= 0) {
        rc = launch_gemv_mma(ml, ts, K, x, x_dtype, ts[0].cols, y, ts[0].rows, RWKVQ_EPI_NONE, nullptr, 1,
                             static_cast<cudaStream_t>(stream));
        return rc ? rc : check_launch("rwkvq_gemv_fused(mma)");
    }
    const int ck = chunk_kind_of(ts[0]);
    RWKVQ_REQUIRE(ck >= 0, RWKVQ_E_DTYPE, "rwkvq_gemv_fused: layout has no chunk kernel");
    GemvArgs a{};
    for (int k = 0; k < K; ++k) a.t[k] = make_view(ts[k]);
    a.x = x; a.x_dtype = x_dtype; a.ldx = ts[0].cols; a.y = y; a.ldy = ts[0].rows;
    a.epilogue = RWKVQ_EPI_NONE; a.n_cols = 1; a.fused = 1;
    // same rows-per-warp as the single-matrix launch: identical summation order
    dispatch_kind<1>(ck, a, ts[0].rows, K, rows_per_warp(ts[0], 1), static_cast<cudaStream_t>(stream));
    return check_launch("rwkvq_gemv_fused");
}

int rwkvq_outlier_tail(const int32_t* row_ptr, const int32_t* cols, const float* delta, int rows, const void* x,
                       int x_dtype, int N, int64_t ldx, float* y, int64_t ldy, int epilogue, const float* resid, void* stream) {
    RWKVQ_REQUIRE(row_ptr && cols && delta && x && y, RWKVQ_E_NULL, "rwkvq_outlier_tail: null pointer");
    RWKVQ_REQUIRE(rows >= 1 && N >= 1 && ldy >= rows, RWKVQ_E_SHAPE, "rwkvq_outlier_tail: rows %d, N %d, ldy %lld", rows, N, (long long)ldy);
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F32 || x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_DTYPE, "rwkvq_outlier_tail: x_dtype %d", x_dtype);
    RWKVQ_REQUIRE(epilogue >= RWKVQ_EPI_NONE && epilogue <= RWKVQ_EPI_ADD, RWKVQ_E_DTYPE, "rwkvq_outlier_tail: epilogue %d", epilogue);
    RWKVQ_REQUIRE(epilogue != RWKVQ_EPI_ADD || resid != nullptr, RWKVQ_E_NULL, "rwkvq_outlier_tail: resid is null");
    const long long total = static_cast<long long>(rows) * N;
    rwkvq::outlier_tail_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        row_ptr, cols, delta, x, x_dtype, ldx, y, ldy, resid, epilogue, rows, N);
    return check_launch("rwkvq_outlier_tail");
}

}  // extern "C"
