// Shared device helpers: streaming loads, the .rwkvq bit layouts as index
// arithmetic, and host-side error plumbing of the C ABI.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "rwkvq_b200.h"

namespace rwkvq {

// ---------------------------------------------------------------- host side
void set_error_detail(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);

#define RWKVQ_REQUIRE(cond, code, ...)                    \
    do {                                                  \
        if (!(cond)) return ::rwkvq::fail((code), __VA_ARGS__); \
    } while (0)

// Launch with programmatic stream serialization: the kernel may start while its
// predecessor in the stream is still draining; it must execute pdl_wait() before it
// reads anything the predecessor wrote and before its first global write.
// RWKVQ_PDL=0 in the environment turns the attribute off.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

static inline bool aligned(const void* p, size_t a) {
    return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

// -------------------------------------------------------------- device side

// Programmatic dependent launch: no-ops when the launch did not opt in.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

// Weights are read exactly once per launch: bypass L1 allocation so that the
// activation vector stays cached.
__device__ __forceinline__ uint4 ld_stream_u128(const void* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_u64(const void* p) {
    uint2 v;
    asm("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                 : "=r"(v.x), "=r"(v.y)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u32(const void* p) {
    uint32_t v;
    asm("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u16(const void* p) {
    uint16_t v;
    asm("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u8(const void* p) {
    uint32_t v;
    asm("ld.global.nc.L1::no_allocate.u8 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}
// fp32 -> fp16 (round to nearest even) -> fp32: the block scale / min are
// defined through this round trip (formats/codec.py:213-215, 255-257).
__device__ __forceinline__ float half_roundtrip(float x) {
    return __half2float(__float2half_rn(x));
}
__device__ __forceinline__ float bf16_roundtrip(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}
// fp16(bf16(x)) as fp32: the reference's load-time rounding of every tensor
// that is not a quantized linear (quant_model.py:128-154 over reader.py:114-127).
__device__ __forceinline__ float dense_param_rounding(float x) {
    return half_roundtrip(bf16_roundtrip(x));
}

// Value i of a little-endian 6-bit stream held in 6 bytes (8 values).
__device__ __forceinline__ uint32_t sixbit(uint64_t stream48, int i) {
    return static_cast<uint32_t>(stream48 >> (6 * i)) & 63u;
}

// sb6 block scale and min for block j (0..7) of a super-block whose 12 metadata
// bytes are m0,m1,m2 (little-endian words): bytes 0-5 carry eight 6-bit scale
// codes, bytes 6-11 eight 6-bit min codes stored +31 (formats/codec.py:208-215).
__device__ __forceinline__ void sb6_scale_min(uint32_t m0, uint32_t m1, uint32_t m2, int j,
                                              float d, float dm, float& s, float& m) {
    const uint64_t qs_stream = static_cast<uint64_t>(m0) | (static_cast<uint64_t>(m1 & 0xFFFFu) << 32);
    const uint64_t qm_stream = static_cast<uint64_t>(m1 >> 16) | (static_cast<uint64_t>(m2) << 16);
    const float qs = static_cast<float>(sixbit(qs_stream, j));
    const float qm = static_cast<float>(static_cast<int>(sixbit(qm_stream, j)) - 31);
    s = fmaxf(half_roundtrip(__fmul_rn(qs, d)), 1e-8f);
    m = half_roundtrip(__fmul_rn(qm, dm));
}

// Spread the 4 bits of `nib` to bit `BIT` of the 4 bytes of a word (bit k of
// nib -> byte k).  The shifted copies of nib occupy disjoint bit ranges, so the
// product has no carries.
template <int BIT>
__device__ __forceinline__ uint32_t spread_nibble(uint32_t nib) {
    return (nib * (0x00204081u << BIT)) & (0x01010101u << BIT);
}

// A float whose bit pattern is byte `k` of `w`: the subnormal k_byte * 2^-149.
// Multiplying by an activation pre-scaled by 2^64 gives an exact product in
// the normal range, so integer codes enter an FFMA without an int->float
// conversion.
template <int K>
__device__ __forceinline__ float byte_as_subnormal(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0u, 0x4440u | K));
}

constexpr float kXPreScale = 0x1p64f;     // activations are staged as x * 2^64
constexpr float kCodeUnscale = 0x1p85f;   // 2^149 / 2^64

// ---- generic per-element decode (dequant kernels, ragged-shape GEMV) --------
struct QView {
    int kind, bits, rows, cols, gs, sb;
    const uint8_t* codes;
    const uint8_t* qh;
    const uint8_t* qh2;
    const uint8_t* qsqm;
    const int8_t* qs;
    const __half* d;
    const __half* dm;
    const void* scale;
    const float* mn;
    const uint8_t* dev_meta;
    const uint32_t* dev_planes;
};

__host__ inline QView make_view(const rwkvq_qtensor& t) {
    QView v;
    v.kind = t.kind; v.bits = t.bits; v.rows = t.rows; v.cols = t.cols; v.gs = t.gs; v.sb = t.sb;
    v.codes = static_cast<const uint8_t*>(t.codes);
    v.qh = static_cast<const uint8_t*>(t.qh);
    v.qh2 = static_cast<const uint8_t*>(t.qh2);
    v.qsqm = static_cast<const uint8_t*>(t.qsqm);
    v.qs = static_cast<const int8_t*>(t.qs);
    v.d = static_cast<const __half*>(t.d);
    v.dm = static_cast<const __half*>(t.dm);
    v.scale = t.scale;
    v.mn = static_cast<const float*>(t.mn);
    v.dev_meta = static_cast<const uint8_t*>(t.dev_meta);
    v.dev_planes = static_cast<const uint32_t*>(t.dev_planes);
    return v;
}

// Low-4-bit code of column c in the block-local split nibble layout
// (formats/codec.py:136-157): inside a block of gs columns, byte j holds column j
// (low nibble) and column j + gs/2 (high nibble).
__device__ __forceinline__ uint32_t blocklocal_nibble(const uint8_t* row_codes, int c, int gs) {
    const int j = c % gs, h = gs >> 1;
    const uint32_t b = row_codes[(c / gs) * h + (j % h)];
    return (j >= h) ? (b >> 4) : (b & 0xFu);
}
__device__ __forceinline__ uint32_t plane_bit(const uint8_t* row_plane, int c) {
    return (row_plane[c >> 3] >> (c & 7)) & 1u;
}

// Exact fp32 value of element (r, c): multiply and add are separate roundings,
// as in the numpy codec.
__device__ __forceinline__ float decode_element(const QView& t, int r, int c) {
    const size_t R = static_cast<size_t>(r);
    switch (t.kind) {
        case RWKVQ_KIND_SB6: {
            const int nsb = t.cols / (t.gs * t.sb);
            const int blk = c / t.gs, sbi = blk / t.sb, j = blk % t.sb;
            uint32_t q = blocklocal_nibble(t.codes + R * (t.cols / 2), c, t.gs);
            if (t.qh) q += 16u * plane_bit(t.qh + R * (t.cols / 8), c);
            if (t.qh2) q += 32u * plane_bit(t.qh2 + R * (t.cols / 8), c);
            const uint8_t* mp = t.qsqm + (R * nsb + sbi) * 12;
            const uint32_t m0 = mp[0] | (mp[1] << 8) | (mp[2] << 16) | (uint32_t(mp[3]) << 24);
            const uint32_t m1 = mp[4] | (mp[5] << 8) | (mp[6] << 16) | (uint32_t(mp[7]) << 24);
            const uint32_t m2 = mp[8] | (mp[9] << 8) | (mp[10] << 16) | (uint32_t(mp[11]) << 24);
            float s, m;
            sb6_scale_min(m0, m1, m2, j, __half2float(t.d[R * nsb + sbi]),
                          __half2float(t.dm[R * nsb + sbi]), s, m);
            return __fadd_rn(__fmul_rn(static_cast<float>(q), s), m);
        }
        case RWKVQ_KIND_SYM: {
            const int nb = t.cols / t.gs, nsb = nb / t.sb;
            const int blk = c / t.gs;
            float q;
            if (t.bits == 8) {
                q = static_cast<float>(reinterpret_cast<const int8_t*>(t.codes)[R * t.cols + c]);
            } else {
                int u = static_cast<int>(blocklocal_nibble(t.codes + R * (t.cols / 2), c, t.gs));
                if (t.qh) u += 16 * static_cast<int>(plane_bit(t.qh + R * (t.cols / 8), c));
                if (t.qh2) u += 32 * static_cast<int>(plane_bit(t.qh2 + R * (t.cols / 8), c));
                q = static_cast<float>(u - 32);
            }
            const float s = half_roundtrip(__fmul_rn(static_cast<float>(t.qs[R * nb + blk]),
                                                     __half2float(t.d[R * nsb + blk / t.sb])));
            return __fmul_rn(q, s);
        }
        case RWKVQ_KIND_ASYM: {
            const int nb = (t.cols + t.gs - 1) / t.gs, blk = c / t.gs;
            const float q = static_cast<float>(t.codes[R * t.cols + c]);
            return __fadd_rn(__fmul_rn(q, static_cast<const float*>(t.scale)[R * nb + blk]),
                             t.mn[R * nb + blk]);
        }
        case RWKVQ_KIND_RTN: {
            int code;
            if (t.bits <= 4) {
                const int half = (t.cols + 1) / 2;
                const bool hi = c >= half;
                const uint32_t b = t.codes[R * half + (hi ? c - half : c)];
                code = static_cast<int>(hi ? (b >> 4) : (b & 0xFu)) - 8;
            } else {
                code = reinterpret_cast<const int8_t*>(t.codes)[R * t.cols + c];
            }
            return __fmul_rn(static_cast<float>(code),
                             __half2float(static_cast<const __half*>(t.scale)[R]));
        }
        default: {   // dense bf16
            return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(t.codes)[R * t.cols + c]);
        }
    }
}

int validate_qtensor(const rwkvq_qtensor* t, const char* who);

// Single-vector tensor-core GEMV (rwkvq_gemv_mma.cu): layout id >= 0 when the
// tensor carries what that kernel needs, and its launcher.
int mma_layout_of(const rwkvq_qtensor& t);
int launch_gemv_mma(int layout, const rwkvq_qtensor* ts, int n_mats, const void* x, int x_dtype,
                    long long ldx, float* y, long long ldy, int epilogue, const float* resid,
                    int fused, cudaStream_t s, const void* const* x_each = nullptr, float* scratch = nullptr);
size_t gemv_mma_scratch_bytes();
// Small-batch tensor-core kernel (rwkvq_gemv_batch.cu): n_mats same-shape matrices, each with its
// own [N, ldx] input and [N, ldy] output; weights read once for all N right-hand sides.  Inputs are
// fp32 rows with scales[k] = max|x| of every row (written by the producer of x or by launch_row_amax),
// or (half_in) fp16 rows already multiplied per row by a power of two with scales[k] = its inverse.
// amax_outs (optional, per matrix): [N] slots the kernel merges max|y| per token into (atomic max on
// the bit pattern; zero them before the launch).
int launch_gemv_batch(const rwkvq_qtensor* ts, int n_mats, const void* const* xs, bool half_in, const float* const* scales,
                      int N, long long ldx, float* const* ys, long long ldy, int epilogue, const float* const* resids,
                      float* const* amax_outs, cudaStream_t s);
// The same product on the tcgen05 tensor cores (rwkvq_gemm_tcb.cu; sb6 / sym tensors, gemm_tcb_ok);
// status: device word that receives RWKVQ_E_TIMEOUT if a bounded pipeline wait ran out.
bool gemm_tcb_ok(const rwkvq_qtensor& t);
bool batch_fast();        // RWKVQ_BATCH_FAST=1: single fp16 operands in the small-batch linears (faster, ~5e-4 per linear)
bool tcb_enabled();
bool tcb_forced();        // a profiling override asks for the tcgen05 kernel at every batch size
int launch_gemm_tcb(const rwkvq_qtensor* ts, int n_mats, const void* const* xs, bool half_in, const float* const* scales,
                    int N, long long ldx, float* const* ys, long long ldy, int epilogue, const float* const* resids,
                    float* const* amax_outs, int* status, cudaStream_t s, bool exact = false,
                    const void* const* xs_lo = nullptr, const void* const* xs_sum = nullptr);   // exact: two-term operands
// LoRA pair of the time-mix block for a batch of streams on the tensor cores (rwkvq_lora_mma.cu)
bool lora_mma_ok(const rwkvq_qtensor* const* t1, const rwkvq_qtensor* const* t2, int n_br, int D);
int launch_lora_pair_mma(const rwkvq_qtensor* const* t1, const rwkvq_qtensor* const* t2, const float* const* xs,
                         float* const* ys, const int* acts, int n_br, int B, int D, int max_rank, float* h, int n_stride,
                         cudaStream_t s);
int launch_row_amax(const float* x, long long ldx, int cols, int N, float* amax, int* status, cudaStream_t s);

}  // namespace rwkvq
