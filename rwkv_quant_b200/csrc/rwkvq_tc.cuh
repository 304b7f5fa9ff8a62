// Device-side building blocks shared by the tcgen05 kernels (rwkvq_gemm_tc.cu: prefill and large
// batches; rwkvq_gemm_tcb.cu: small decode batches): PTX wrappers for mbarriers, tensor memory and
// tcgen05.mma, the 128-byte-swizzled K-major operand layout, and the weight producer that turns
// packed file bytes into fp16 operand rows.
#pragma once
#include <cuda.h>

#include "rwkvq_common.cuh"

namespace rwkvq {

constexpr int kGmRows = 128;          // output rows per CTA (UMMA M)
constexpr int kGmK = 64;              // K per slab: one 128-byte swizzle row of fp16
constexpr unsigned kGmSpinLimit = 1u << 24;
// upper bound of one suspended try_wait: without it a waiter that went to sleep before the phase
// completed was seen to wake only after ~10 us
constexpr unsigned kGmSuspendNs = 256;

// ---- PTX wrappers ---------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    const uint32_t a = smem_addr(bar);
    for (unsigned i = 0; i < kGmSpinLimit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(a), "r"(parity), "r"(kGmSuspendNs)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// 2-D tile load, this CTA's shared memory only (no multicast)
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_addr(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_addr(bar))
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(dst_smem)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// K-major operand tile, 128-byte swizzle: row r (128 bytes = 64 fp16) sits in the
// 1024-byte atom r/8; its 16-byte chunk c is stored at chunk position c ^ (r % 8).
__device__ __forceinline__ uint32_t sw128_offset(int r, int chunk) {
    return static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4));
}
// Shared-memory matrix descriptor: start address, leading offset (unused for a
// swizzled K-major tile), stride between 8-row atoms = 1024 bytes, version 1, SWIZZLE_128B.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(1) << 16) |
           (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) |
           (static_cast<uint64_t>(2) << 61);
}
// Instruction descriptor of kind::f16: D = f32, A = B = fp16, both K-major, M = 128, N.
__device__ __forceinline__ uint32_t umma_idesc(int n) {
    return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kGmRows >> 4) << 24);
}

// ---- weight producer ----------------------------------------------------------------
// One macro-iteration covers K = 256 (one super-block): four 64-K slabs of the A operand.
// The 128 rows x 8 items (32 columns each) of a macro-iteration are spread over the 256
// producer threads so that the 8 lanes of a row read the row's packed super-block as one
// contiguous run (128 B of nibble codes / 256 B of int8 codes, 32 B of each bit-plane, one
// 16-byte scale record): item q of thread tid is (row 32 q + tid / 8, item tid % 8).

// 4 code bytes of a word -> 4 fp16 = fp16(code * s + m), two HFMA2.  `bias` is the value
// to subtract from (1024 + byte): 1024 for unsigned codes, 1056 / 1152 for codes stored
// +32 / bytes biased by 128.
__device__ __forceinline__ uint2 bytes_to_half4(uint32_t w, __half2 bias, __half2 s2, __half2 m2) {
    const uint32_t lo = __byte_perm(w, 0x64646464u, 0x4140), hi = __byte_perm(w, 0x64646464u, 0x4342);
    const __half2 a = __hfma2(__hsub2(*reinterpret_cast<const __half2*>(&lo), bias), s2, m2);
    const __half2 b = __hfma2(__hsub2(*reinterpret_cast<const __half2*>(&hi), bias), s2, m2);
    return make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

// Packed bytes of one item: 32 consecutive weights of one row.
struct Packed {
    uint4 c0, c1;          // codes (c1: second 16 bytes of int8 layouts)
    uint32_t h, h2;        // bit-plane words of the 32 columns
    uint4 rec;             // sb6: 16-byte scale record (relayouted) or {m0, m1, m2, d | dm << 16} from the file
                           // sym: .x = two int8 scale codes, .y = d
};

// item `it` (0..7) of super-block `sbk` of row `row_g`
__device__ __forceinline__ void load_packed(Packed& p, const QView& t, int row_g, int sbk, int it) {
    const size_t R = static_cast<size_t>(row_g);
    const int nsb = t.cols >> 8;
    const int c0 = sbk * 256 + it * 32;
    p.h = p.h2 = 0;
    if (t.kind == RWKVQ_KIND_SB6) {
        p.c0 = ld_stream_u128(t.codes + R * (t.cols >> 1) + (c0 >> 1));
        if (t.qh) p.h = ld_stream_u32(t.qh + R * (t.cols >> 3) + (c0 >> 3));
        if (t.qh2) p.h2 = ld_stream_u32(t.qh2 + R * (t.cols >> 3) + (c0 >> 3));
        if (t.dev_meta) {
            p.rec = ld_stream_u128(t.dev_meta + (R * nsb + sbk) * 16);
        } else {
            const uint8_t* mp = t.qsqm + (R * nsb + sbk) * 12;
            p.rec.x = ld_stream_u32(mp); p.rec.y = ld_stream_u32(mp + 4); p.rec.z = ld_stream_u32(mp + 8);
            p.rec.w = ld_stream_u16(t.d + R * nsb + sbk) | (ld_stream_u16(t.dm + R * nsb + sbk) << 16);
        }
    } else {
        p.rec.y = ld_stream_u16(t.d + R * nsb + sbk);
        p.rec.x = ld_stream_u16(t.qs + R * (t.cols >> 4) + (c0 >> 4));
        if (t.bits == 8) {
            const uint8_t* cp = t.codes + R * t.cols + c0;
            p.c0 = ld_stream_u128(cp); p.c1 = ld_stream_u128(cp + 16);
        } else {
            p.c0 = ld_stream_u128(t.codes + R * (t.cols >> 1) + (c0 >> 1));
            p.h = ld_stream_u32(t.qh + R * (t.cols >> 3) + (c0 >> 3));
            p.h2 = ld_stream_u32(t.qh2 + R * (t.cols >> 3) + (c0 >> 3));
        }
    }
}

// The 32 codes of an item as bytes with their block scales and mins.
struct ItemCodes {
    uint32_t bytes[8];                             // column order
    __half2 s2[2], m2[2], bias;                    // per 16 columns; bias: see bytes_to_half4
};

// `it` = item index inside the super-block (selects the block scales), `half` = it % 2.
__device__ __forceinline__ void decode_item(const Packed& p, const QView& t, int it, int half, ItemCodes& c) {
    uint32_t (&bytes)[8] = c.bytes;
    __half2 (&s2)[2] = c.s2;
    __half2 (&m2)[2] = c.m2;
    __half2& bias = c.bias;
    const uint32_t h = p.h, h2 = p.h2;
    if (t.kind == RWKVQ_KIND_SB6) {
        const uint32_t w[4] = {p.c0.x, p.c0.y, p.c0.z, p.c0.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {              // byte k of the block: column k (low), k + 16 (high)
            bytes[i] = w[i] & 0x0F0F0F0Fu;
            bytes[4 + i] = (w[i] >> 4) & 0x0F0F0F0Fu;
        }
        if (t.qh) {                                // uniform over the launch: 4-bit tensors skip the plane work
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                bytes[i] |= spread_nibble<4>((h >> (4 * i)) & 0xFu);
                bytes[4 + i] |= spread_nibble<4>((h >> (16 + 4 * i)) & 0xFu);
            }
        }
        if (t.qh2) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                bytes[i] |= spread_nibble<5>((h2 >> (4 * i)) & 0xFu);
                bytes[4 + i] |= spread_nibble<5>((h2 >> (16 + 4 * i)) & 0xFu);
            }
        }
        float s, m;
        if (t.dev_meta) {
            // record word it/2: 6-bit scale codes of blocks 2(it/2), 2(it/2)+1, min codes (+31), one byte of d | dm << 16
            const int tt = it >> 1;
            const uint32_t w4 = (tt & 2) ? ((tt & 1) ? p.rec.w : p.rec.z) : ((tt & 1) ? p.rec.y : p.rec.x);
            const uint32_t dd = __byte_perm(p.rec.x, p.rec.y, 0x0073) & 0xFFFFu;     // d
            const uint32_t dm = __byte_perm(p.rec.z, p.rec.w, 0x0073) & 0xFFFFu;     // dm
            const float qs = static_cast<float>((w4 >> (6 * half)) & 0x3Fu);
            const float qm = static_cast<float>(static_cast<int>((w4 >> (12 + 6 * half)) & 0x3Fu) - 31);
            s = fmaxf(half_roundtrip(__fmul_rn(qs, half_bits_to_float(dd))), 1e-8f);
            m = half_roundtrip(__fmul_rn(qm, half_bits_to_float(dm)));
        } else {
            sb6_scale_min(p.rec.x, p.rec.y, p.rec.z, it, half_bits_to_float(p.rec.w & 0xFFFFu),
                          half_bits_to_float(p.rec.w >> 16), s, m);
        }
        s2[0] = s2[1] = __float2half2_rn(s);
        m2[0] = m2[1] = __float2half2_rn(m);
        bias = __float2half2_rn(1024.f);
    } else {                                       // sym: two blocks of 16
        const float d = half_bits_to_float(p.rec.y);
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const int q = static_cast<int8_t>((p.rec.x >> (8 * b)) & 0xFFu);
            s2[b] = __float2half2_rn(half_roundtrip(__fmul_rn(static_cast<float>(q), d)));
            m2[b] = __float2half2_rn(0.f);
        }
        if (t.bits == 8) {
            const uint32_t w[8] = {p.c0.x, p.c0.y, p.c0.z, p.c0.w, p.c1.x, p.c1.y, p.c1.z, p.c1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) bytes[i] = w[i] ^ 0x80808080u;      // code + 128
            bias = __float2half2_rn(1152.f);
        } else {
            const uint32_t w[4] = {p.c0.x, p.c0.y, p.c0.z, p.c0.w};
#pragma unroll
            for (int b = 0; b < 2; ++b)            // block b: words 2b, 2b+1; byte k: column k (low), k + 8 (high)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int cl = 16 * b + 4 * i, ch = cl + 8;
                    bytes[4 * b + i] = (w[2 * b + i] & 0x0F0F0F0Fu) | spread_nibble<4>((h >> cl) & 0xFu) |
                                       spread_nibble<5>((h2 >> cl) & 0xFu);
                    bytes[4 * b + 2 + i] = ((w[2 * b + i] >> 4) & 0x0F0F0F0Fu) | spread_nibble<4>((h >> ch) & 0xFu) |
                                           spread_nibble<5>((h2 >> ch) & 0xFu);
                }
            bias = __float2half2_rn(1056.f);       // stored code = value + 32
        }
    }
}

// 32 weights -> fp16, stored as 4 swizzled 16-byte chunks of row r: chunks 4*half .. +3 of the slab.
__device__ __forceinline__ void convert_store(const Packed& p, const QView& t, int r, int it, int half,
                                              unsigned char* a_slab) {
    ItemCodes c;
    decode_item(p, t, it, half, c);
#pragma unroll
    for (int j = 0; j < 4; ++j) {                  // chunk j: columns 8j .. 8j+7 of the 32
        const uint2 a = bytes_to_half4(c.bytes[2 * j], c.bias, c.s2[j >> 1], c.m2[j >> 1]);
        const uint2 b = bytes_to_half4(c.bytes[2 * j + 1], c.bias, c.s2[j >> 1], c.m2[j >> 1]);
        *reinterpret_cast<uint4*>(a_slab + sw128_offset(r, 4 * half + j)) = make_uint4(a.x, a.y, b.x, b.y);
    }
}

// 4 code bytes -> the product code * s as TWO fp16 terms: p = fp16(code * s) and the rounding error
// of that product, which a fused multiply-add recovers exactly (code * s has at most 19 significant
// bits, p keeps the top 11): p + e = code * s up to the fp16 subnormal quantum (6e-8 absolute).
__device__ __forceinline__ void bytes_to_half4_pair(uint32_t w, __half2 bias, __half2 s2, uint2& p, uint2& e) {
    const uint32_t lo = __byte_perm(w, 0x64646464u, 0x4140), hi = __byte_perm(w, 0x64646464u, 0x4342);
    const __half2 q01 = __hsub2(*reinterpret_cast<const __half2*>(&lo), bias);
    const __half2 q23 = __hsub2(*reinterpret_cast<const __half2*>(&hi), bias);
    const __half2 p01 = __hmul2(q01, s2), p23 = __hmul2(q23, s2);
    const __half2 e01 = __hfma2(q01, s2, __hneg2(p01)), e23 = __hfma2(q23, s2, __hneg2(p23));
    p = make_uint2(*reinterpret_cast<const uint32_t*>(&p01), *reinterpret_cast<const uint32_t*>(&p23));
    e = make_uint2(*reinterpret_cast<const uint32_t*>(&e01), *reinterpret_cast<const uint32_t*>(&e23));
}

// convert_store with the products code * s as two terms: p into a_slab, e into e_slab (same
// positions).  The block min is NOT folded in: it is returned (an fp16 value by the codec's
// definition; zero for the layouts without one) and multiplies the block's activation sum instead.
__device__ __forceinline__ __half convert_store_pair(const Packed& p, const QView& t, int r, int it, int half,
                                                     unsigned char* a_slab, unsigned char* e_slab) {
    ItemCodes c;
    decode_item(p, t, it, half, c);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint2 pa, ea, pb, eb;
        bytes_to_half4_pair(c.bytes[2 * j], c.bias, c.s2[j >> 1], pa, ea);
        bytes_to_half4_pair(c.bytes[2 * j + 1], c.bias, c.s2[j >> 1], pb, eb);
        const uint32_t off = sw128_offset(r, 4 * half + j);
        *reinterpret_cast<uint4*>(a_slab + off) = make_uint4(pa.x, pa.y, pb.x, pb.y);
        *reinterpret_cast<uint4*>(e_slab + off) = make_uint4(ea.x, ea.y, eb.x, eb.y);
    }
    return __low2half(c.m2[0]);
}

// Shared-memory matrix descriptor of a K-major operand without swizzle: 8 rows x 16 bytes form a
// contiguous core matrix; `kstep` bytes lead from one core matrix to the next along K, `mstep`
// bytes to the next group of 8 rows.
__device__ __forceinline__ uint64_t umma_desc_plain(uint32_t saddr, uint32_t kstep, uint32_t mstep) {
    return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(kstep >> 4) << 16) |
           (static_cast<uint64_t>(mstep >> 4) << 32) | (static_cast<uint64_t>(1) << 46);
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

}  // namespace rwkvq
