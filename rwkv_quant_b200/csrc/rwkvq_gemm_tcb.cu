// Quantized linear for a small batch of right-hand sides (decode streams) on the tcgen05 tensor
// cores:   y[n, o] = epi( sum_c W[o, c] x[n, c] ),   n < N <= 64 per token group.
//
// The mma.sync form of this product (rwkvq_gemv_batch.cu) issues one warp-level MMA per 16 rows x
// 8 tokens x 16 columns plus a shared-memory load and a share of the code -> fp16 conversion, and
// on this part those issue slots add up instead of overlapping.  Here a CTA owns 128 output rows
// (the UMMA M) and all tokens of its group (UMMA N = 16, 32 or 64):
//   * 8 producer warps read the packed rows of a 256-column pass exactly as the prefill kernel
//     does (load_packed: one contiguous run per row), one pass ahead in registers, turn them into
//     fp16(q*s + m) and store them K-major with the 128-byte swizzle (convert_store);
//   * the same warps stage the activations of the pass: fp16 rows already scaled per token (from
//     the LayerNorm kernels) are copied, fp32 rows are scaled by the power of two their known
//     max|x| implies and rounded once; both land in the swizzled K-major layout the tensor core
//     reads, written with plain stores (no tensor map);
//   * one lane of a ninth warp issues the 16 tcgen05.mma (M 128, N tokens, K 16) of the pass into
//     a tensor-memory accumulator and commits them to the mbarrier the producers wait on before
//     they overwrite the operands;
//   * the K loop is split over a thread-block cluster (up to 8 CTAs); the accumulator goes
//     through tcgen05.ld into shared memory (over the dead operand buffers), and after one
//     cluster barrier every CTA adds a slice of the tile over all ranks through distributed
//     shared memory in rank order, applies the epilogue and stores.
// Every mbarrier wait is bounded; on expiry the CTA records RWKVQ_E_TIMEOUT in the status word,
// skips its work, still passes the cluster barriers, frees its tensor memory and returns.
// A second form of the kernel (template parameter EX, described at the kernel) keeps both operands
// as two fp16 terms and gives fp32-grade results.
#include <cooperative_groups.h>

#include <stdlib.h>

#include <algorithm>

#include "rwkvq_tc.cuh"

namespace cg = cooperative_groups;

namespace rwkvq {

constexpr int kTbProducers = 256;         // warps 0-7: weights, activations, epilogue
constexpr int kTbThreads = 288;           // + warp 8: one lane issues the MMAs
constexpr int kTbSbK = 256;               // columns of a super-block
constexpr int kTbRP = kGmRows + 4;        // pitch of a partial-sum row
constexpr int kTbMaxMats = 4;
extern unsigned long long* g_batch_trace;      // rwkvq_gemv_batch.cu: set by rwkvq_profiling_batch_trace

struct TcbArgs {
    QView t[kTbMaxMats];
    const float* x[kTbMaxMats];           // [N, ldx] fp32, or null when x16 is given
    const float* amax[kTbMaxMats];        // with x:   [N] max|x| per token
    const __half* x16[kTbMaxMats];        // [N, ldx] fp16 rows = x * 2^s
    const __half* x16lo[kTbMaxMats];      // two-term kernel with x16: fp16(x * 2^s - x16)
    const __half* xsum[kTbMaxMats];       // ... and [N, cols / 128][8]: the sums of x * 2^s over the four 32-column blocks
                                          //     of every 128 columns, 4 high halves then 4 low halves
    const float* unscale[kTbMaxMats];     // with x16: [N] 2^-s
    float* y[kTbMaxMats];                 // [N, ldy]
    const float* resid[kTbMaxMats];
    float* amax_out[kTbMaxMats];          // optional [N]: max|y| per token is merged into it (atomic max; zeroed by the caller)
    long long ldx, ldy;
    int n_tokens, epilogue;
    int passes;                           // passes of one CTA's K slice: 256 columns each, 128 in the two-term kernel
    int ks;                               // CTAs along K = cluster size
    int* status;                          // device word: first error code, 0 = ok
    unsigned long long* trace;            // profiling aid (rwkvq_profiling.h): global-timer marks of CTA (0,0,0), or null
};

__device__ __forceinline__ void tb_mark(const TcbArgs& a, int slot) {
    if (a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        a.trace[slot] = t;
    }
}

// EX: both operands as two fp16 terms (W: p = fp16(q*s) and its exact rounding error e; x: hi =
// fp16(x * 2^s) and lo = fp16(x * 2^s - hi)) and three MMAs per K step (e*hi + p*lo + p*hi) into the
// one accumulator; the block mins, fp16 values by the codec's definition, multiply the per-block
// sums of the activations in one more MMA per pass (K = the 4 blocks of the pass against their high
// halves + the same 4 against their low halves, in a small operand pair without swizzle).  The fp32
// accumulation is then the only rounding that matters (~1e-6 against an fp32 dequantise-and-multiply
// instead of ~5e-4).  A pass covers 128 columns so that the doubled operands keep the shared-memory
// footprint of the single-term form; the activations are scaled to at most 2^9 so that a block sum
// stays inside the fp16 range.
template <int NT, bool EX>
__global__ void __launch_bounds__(kTbThreads, 2) gemm_tcb_kernel(const TcbArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int PASSK = EX ? 128 : 256;                        // columns of a pass
    constexpr int SLABS = PASSK / kGmK;                          // 64-K slabs of a pass: 2 or 4
    constexpr int ITEMS = PASSK / 32;                            // 32-column items of a row and pass: 4 or 8
    constexpr int RGRP = kTbProducers / ITEMS;                   // rows one item per thread covers: 64 or 32
    constexpr int QN = kGmRows / RGRP;                           // items per thread and pass: 2 or 4
    constexpr int SLAB = kGmRows * 128, BSLAB = NT * 128;
    constexpr uint32_t TM_COLS = NT < 32 ? 32 : NT;
    constexpr int RP = kTbRP;
    unsigned char* a_slabs = smem;                               // [SLABS][SLAB]  weights of the pass (EX: p)
    unsigned char* e_slabs = a_slabs + SLABS * SLAB;             // EX: [SLABS][SLAB] e
    unsigned char* b_slabs = a_slabs + (EX ? 2 : 1) * SLABS * SLAB;   // [SLABS][BSLAB] activations of the pass (EX: hi)
    unsigned char* l_slabs = b_slabs + SLABS * BSLAB;            // EX: [SLABS][BSLAB] lo
    unsigned char* m_a = l_slabs + SLABS * BSLAB;                // EX: [2][128 rows][16 B] block mins (K 0-3 and again 4-7; K 8-15 zero)
    unsigned char* m_b = m_a + 2 * kGmRows * 16;                 // EX: [2][NT][16 B] block sums (4 high, 4 low halves; K 8-15 zero)
    const bool has_min = EX && a.t[blockIdx.y].kind == RWKVQ_KIND_SB6;
    float* part = reinterpret_cast<float*>(a_slabs);             // [NT][RP], over the operands once the MMAs are done
    __shared__ uint64_t bar_full, bar_mma;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_fail;
    __shared__ float s_sc[NT], s_un[NT], s_omax[NT];
    cg::cluster_group cluster = cg::this_cluster();

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const QView& t = a.t[blockIdx.y];
    const int ks = a.ks, rank = static_cast<int>(blockIdx.x) % ks, rt = static_cast<int>(blockIdx.x) / ks;
    const int row0 = rt * kGmRows;
    const int n0 = blockIdx.z * NT, nn = min(NT, a.n_tokens - n0);
    const int np = a.passes, pass0 = rank * np;                 // first pass of this CTA, in units of PASSK columns
    const bool is16 = a.x16[blockIdx.y] != nullptr;

    tb_mark(a, 0);
    if (tid == 0) {
        mbar_init(&bar_full, kTbProducers / 32);
        mbar_init(&bar_mma, 1);
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    pdl_launch_dependents();
    if (warp == 0) tmem_alloc(&s_tmem, TM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    tb_mark(a, 1);

    if (warp == kTbProducers / 32) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            pdl_wait();
            const uint32_t idesc = umma_idesc(NT);
            const uint64_t a_desc0 = umma_desc(smem_addr(a_slabs)), b_desc0 = umma_desc(smem_addr(b_slabs));
            const uint64_t e_desc0 = umma_desc(smem_addr(e_slabs)), l_desc0 = umma_desc(smem_addr(l_slabs));
            const uint64_t ma_desc = umma_desc_plain(smem_addr(m_a), kGmRows * 16, 128);
            const uint64_t mb_desc = umma_desc_plain(smem_addr(m_b), NT * 16, 128);
            bool ok = true;
            for (int p = 0; p < np && ok; ++p) {
                if (!mbar_wait_bounded(&bar_full, p & 1)) { ok = false; break; }
                if (s_fail) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int sl = 0; sl < SLABS; ++sl) {
                    const uint64_t ad = a_desc0 + (static_cast<uint64_t>(sl * SLAB) >> 4);
                    const uint64_t bd = b_desc0 + (static_cast<uint64_t>(sl * BSLAB) >> 4);
                    const uint64_t ed = e_desc0 + (static_cast<uint64_t>(sl * SLAB) >> 4);
                    const uint64_t ld = l_desc0 + (static_cast<uint64_t>(sl * BSLAB) >> 4);
#pragma unroll
                    for (int k = 0; k < kGmK / 16; ++k) {      // 32 bytes further along K per step
                        if (EX) {                               // small terms first
                            umma_f16(tmem, ed + 2 * k, bd + 2 * k, idesc, (p | sl | k) ? 1u : 0u);
                            umma_f16(tmem, ad + 2 * k, ld + 2 * k, idesc, 1u);
                            umma_f16(tmem, ad + 2 * k, bd + 2 * k, idesc, 1u);
                        } else {
                            umma_f16(tmem, ad + 2 * k, bd + 2 * k, idesc, (p | sl | k) ? 1u : 0u);
                        }
                    }
                }
                if (has_min) umma_f16(tmem, ma_desc, mb_desc, idesc, 1u);
                umma_commit(&bar_mma);
            }
            if (!ok) s_fail = 1;
        }
    } else {
        // ------------------------------------------------------------------ producers
        const int pit = tid % ITEMS, prow = tid / ITEMS;       // item (32 columns) of the pass, row within a group of RGRP
        // packed weights in registers, one pass ahead.  (Two passes ahead in two register sets, i.e. two
        // copies of the pass body, was measured in the two-term kernel: 116 KB of code instead of 64 KB, an
        // instruction-cache hit rate of 74-80 %, and a 64-stream decode step of 4.63 instead of 4.27 ms.)
        constexpr int AHEAD = 1;
        Packed P0[QN];
        // pass p of this CTA: super-block and first item inside it
        auto sb_of = [&](int p) { return EX ? (pass0 + p) >> 1 : pass0 + p; };
        auto item_of = [&](int p) { return EX ? ((pass0 + p) & 1) * ITEMS + pit : pit; };
        auto load_all = [&](int p, Packed* P) {
#pragma unroll
            for (int q = 0; q < QN; ++q) load_packed(P[q], t, min(row0 + RGRP * q + prow, t.rows - 1), sb_of(p), item_of(p));
        };
        load_all(0, P0);                                        // weights do not depend on the producer of x
        pdl_wait();
        tb_mark(a, 2);
        if (tid < NT) {
            float s1 = 1.f, u1 = 1.f;
            if (is16) {
                if (tid < nn) u1 = __ldcg(a.unscale[blockIdx.y] + n0 + tid);
            } else {
                // |x| * 2^(14 - e) <= 2^14 with max|x| <= 2^e; a non-finite row keeps scale 1 and propagates
                const float am = tid < nn ? __ldcg(a.amax[blockIdx.y] + n0 + tid) : 0.f;
                if (am > 0.f && am < INFINITY) {
                    int e = 0;
                    frexpf(am, &e);
                    e = max(-100, e);
                    s1 = ldexpf(1.f, (EX ? 9 : 14) - e);
                    u1 = ldexpf(1.f, e - (EX ? 9 : 14));
                }
            }
            s_sc[tid] = s1; s_un[tid] = u1; s_omax[tid] = 0.f;
        }
        if (has_min) {                                          // the K 8-15 halves of the min operands stay zero
            for (int i = tid; i < kGmRows + NT; i += kTbProducers)
                *reinterpret_cast<uint4*>(i < kGmRows ? m_a + kGmRows * 16 + i * 16 : m_b + NT * 16 + (i - kGmRows) * 16) = make_uint4(0, 0, 0, 0);
        }
        // producers only: named barrier 1 (the issuer warp does not take part)
        asm volatile("bar.sync 1, %0;" ::"n"(kTbProducers) : "memory");
        constexpr int VROW = PASSK / 8;                         // 8-column vectors per token and pass: 32 or 16
        constexpr int VPT = NT * VROW / kTbProducers;           // ... per thread: 2, 4, 8 (EX: 1, 2, 4)
        auto do_pass = [&](int p, Packed* P) {
            const int kbase = (pass0 + p) * PASSK;
            uint4 xv[VPT], xl[EX ? VPT : 1], sv = make_uint4(0, 0, 0, 0);
            if (has_min && is16 && tid < nn)
                sv = __ldcg(reinterpret_cast<const uint4*>(a.xsum[blockIdx.y] + (static_cast<size_t>(n0 + tid) * (t.cols >> 7) + pass0 + p) * 8));
            if (is16) {                                          // requested before the wait and the conversion
                const __half* xg = a.x16[blockIdx.y] + static_cast<size_t>(n0) * a.ldx + kbase;
                const __half* xlg = EX ? a.x16lo[blockIdx.y] + static_cast<size_t>(n0) * a.ldx + kbase : nullptr;
#pragma unroll
                for (int u = 0; u < VPT; ++u) {
                    const int idx = tid + u * kTbProducers, n = idx / VROW, k8 = idx % VROW;
                    xv[u] = n < nn ? __ldcg(reinterpret_cast<const uint4*>(xg + static_cast<size_t>(n) * a.ldx) + k8) : make_uint4(0, 0, 0, 0);
                    if (EX) xl[u] = n < nn ? __ldcg(reinterpret_cast<const uint4*>(xlg + static_cast<size_t>(n) * a.ldx) + k8) : make_uint4(0, 0, 0, 0);
                }
            }
            if (p > 0) {                                         // the MMAs of the previous pass have read the operands
                if (lane == 0 && !s_fail && !mbar_wait_bounded(&bar_mma, (p - 1) & 1)) s_fail = 1;
                __syncwarp();
            }
            if (!__any_sync(0xFFFFFFFFu, s_fail != 0)) {
#pragma unroll
                for (int q = 0; q < QN; ++q) {
                    if (EX) {
                        const __half mn = convert_store_pair(P[q], t, RGRP * q + prow, item_of(p), pit & 1, a_slabs + (pit >> 1) * SLAB,
                                                             e_slabs + (pit >> 1) * SLAB);
                        if (has_min) {                           // block `pit` of the pass: beside the high and the low sums
                            __half* mrow = reinterpret_cast<__half*>(m_a + (RGRP * q + prow) * 16);
                            mrow[pit] = mn;
                            mrow[4 + pit] = mn;
                        }
                    } else {
                        convert_store(P[q], t, RGRP * q + prow, pit, pit & 1, a_slabs + (pit >> 1) * SLAB);
                    }
                }
                if (has_min && is16 && tid < NT) *reinterpret_cast<uint4*>(m_b + tid * 16) = sv;
                if (is16) {
#pragma unroll
                    for (int u = 0; u < VPT; ++u) {
                        const int idx = tid + u * kTbProducers, n = idx / VROW, k8 = idx % VROW;
                        *reinterpret_cast<uint4*>(b_slabs + (k8 >> 3) * BSLAB + sw128_offset(n, k8 & 7)) = xv[u];
                        if (EX) *reinterpret_cast<uint4*>(l_slabs + (k8 >> 3) * BSLAB + sw128_offset(n, k8 & 7)) = xl[u];
                    }
                } else if (EX) {
                    const float* xg = a.x[blockIdx.y] + static_cast<size_t>(n0) * a.ldx + kbase;
                    constexpr int RV = VPT > 1 ? VPT / 2 : 1;     // vectors per round: half of them in flight at a time
#pragma unroll
                    for (int r0 = 0; r0 < VPT; r0 += RV) {
                        float4 f[RV][2];
#pragma unroll
                        for (int u = 0; u < RV; ++u) {
                            const int idx = tid + (r0 + u) * kTbProducers, n = idx / VROW, k8 = idx % VROW;
                            const float4* src = reinterpret_cast<const float4*>(xg + static_cast<size_t>(n) * a.ldx) + 2 * k8;
                            f[u][0] = n < nn ? __ldcg(src) : make_float4(0.f, 0.f, 0.f, 0.f);
                            f[u][1] = n < nn ? __ldcg(src + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int u = 0; u < RV; ++u) {
                            const int idx = tid + (r0 + u) * kTbProducers, n = idx / VROW, k8 = idx % VROW;
                            const float s1 = s_sc[n];
                            const float v[8] = {f[u][0].x * s1, f[u][0].y * s1, f[u][0].z * s1, f[u][0].w * s1,
                                                f[u][1].x * s1, f[u][1].y * s1, f[u][1].z * s1, f[u][1].w * s1};
                            uint32_t hw[4], lw[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const __half2 hh = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
                                const float2 hf = __half22float2(hh);
                                const __half2 ll = __floats2half2_rn(v[2 * j] - hf.x, v[2 * j + 1] - hf.y);
                                hw[j] = *reinterpret_cast<const uint32_t*>(&hh);
                                lw[j] = *reinterpret_cast<const uint32_t*>(&ll);
                            }
                            const uint32_t off = (k8 >> 3) * BSLAB + sw128_offset(n, k8 & 7);
                            *reinterpret_cast<uint4*>(b_slabs + off) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                            *reinterpret_cast<uint4*>(l_slabs + off) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
                            if (has_min) {      // 4 consecutive lanes hold the 32 columns of one block
                                float bs = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
                                bs += __shfl_xor_sync(0xFFFFFFFFu, bs, 1);
                                bs += __shfl_xor_sync(0xFFFFFFFFu, bs, 2);
                                if ((k8 & 3) == 0) {
                                    __half* srow = reinterpret_cast<__half*>(m_b + n * 16);
                                    const __half sh = __float2half_rn(bs);
                                    srow[k8 >> 2] = sh;
                                    srow[4 + (k8 >> 2)] = __float2half_rn(bs - __half2float(sh));
                                }
                            }
                        }
                    }
                } else {
                    const float* xg = a.x[blockIdx.y] + static_cast<size_t>(n0) * a.ldx + kbase;
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {             // two rounds: half the vectors' loads in flight at a time
                        float4 f[VPT / 2 > 0 ? VPT / 2 : 1][2];
#pragma unroll
                        for (int u = 0; u < VPT / 2; ++u) {
                            const int idx = tid + (h2 * (VPT / 2) + u) * kTbProducers, n = idx >> 5, k8 = idx & 31;
                            const float4* src = reinterpret_cast<const float4*>(xg + static_cast<size_t>(n) * a.ldx) + 2 * k8;
                            f[u][0] = n < nn ? __ldcg(src) : make_float4(0.f, 0.f, 0.f, 0.f);
                            f[u][1] = n < nn ? __ldcg(src + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int u = 0; u < VPT / 2; ++u) {
                            const int idx = tid + (h2 * (VPT / 2) + u) * kTbProducers, n = idx >> 5, k8 = idx & 31;
                            const float s1 = s_sc[n];
                            const __half2 h0 = __floats2half2_rn(f[u][0].x * s1, f[u][0].y * s1), h1 = __floats2half2_rn(f[u][0].z * s1, f[u][0].w * s1);
                            const __half2 h2v = __floats2half2_rn(f[u][1].x * s1, f[u][1].y * s1), h3 = __floats2half2_rn(f[u][1].z * s1, f[u][1].w * s1);
                            uint4 pk;
                            pk.x = *reinterpret_cast<const uint32_t*>(&h0); pk.y = *reinterpret_cast<const uint32_t*>(&h1);
                            pk.z = *reinterpret_cast<const uint32_t*>(&h2v); pk.w = *reinterpret_cast<const uint32_t*>(&h3);
                            *reinterpret_cast<uint4*>(b_slabs + (k8 >> 3) * BSLAB + sw128_offset(n, k8 & 7)) = pk;
                        }
                    }
                }
            }
            fence_async_smem();                                 // generic-proxy stores -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_full);              // one arrival per warp
            if (p == 0) tb_mark(a, 3);
            if (p + AHEAD < np) load_all(p + AHEAD, P);         // the registers are free again
        };
#pragma unroll 1
        for (int p = 0; p < np; ++p) do_pass(p, P0);
        // the accumulator is complete when the last commit has arrived
        if (lane == 0 && !s_fail && !mbar_wait_bounded(&bar_mma, (np - 1) & 1)) s_fail = 1;
        __syncwarp();
        tb_mark(a, 4);
    }
    tc_fence_after();
    __syncthreads();
    const bool failed = s_fail != 0;
    if (failed) {
        if (tid == 0 && a.status) atomicCAS(a.status, 0, RWKVQ_E_TIMEOUT);
    } else if (warp < kTbProducers / 32) {
        // warp w reads tensor-memory lanes 32 (w % 4) .. +31 (= output rows); the two warps of a lane group split the tokens
        const int rl = (warp & 3) * 32 + lane;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        for (int c0 = (warp >> 2) * 8; c0 < NT; c0 += 16) {
            float v[8];
            tmem_ld8(lane_base + c0, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) part[(c0 + j) * RP + rl] = v[j] * s_un[c0 + j];
        }
    }
    tc_fence_before();
    tb_mark(a, 5);
    cluster.sync();
    tb_mark(a, 6);
    if (!failed) {
        // ---- add the ks partial tiles in rank order, epilogue, store: float4 groups of 4 rows
        float* y = a.y[blockIdx.y] + static_cast<size_t>(n0) * a.ldy;
        const float* resid = a.resid[blockIdx.y] ? a.resid[blockIdx.y] + static_cast<size_t>(n0) * a.ldy : nullptr;
        const bool vec_io = (a.ldy % 4 == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0) &&
                            (resid == nullptr || (reinterpret_cast<uintptr_t>(resid) & 15) == 0);
        constexpr int g4 = kGmRows / 4;
        const int total4 = nn * g4;
        const int per = (total4 + ks - 1) / ks;
        const int lo = rank * per, hi = min(total4, lo + per);
        for (int i4 = lo + tid; i4 < hi; i4 += kTbThreads) {
            const int n = i4 / g4, r = (i4 - n * g4) * 4;
            const int row = row0 + r;
            if (row >= t.rows) continue;
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int kb = 0; kb < ks; kb += 8) {                // 8 loads in flight, added in rank order
                float4 v[8];
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (kb + k < ks) v[k] = *reinterpret_cast<const float4*>(cluster.map_shared_rank(part, kb + k) + n * RP + r);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (kb + k < ks) { s.x += v[k].x; s.y += v[k].y; s.z += v[k].z; s.w += v[k].w; }
            }
            const size_t o = static_cast<size_t>(n) * a.ldy + row;
            const bool full = vec_io && row + 3 < t.rows;
            if (a.epilogue == RWKVQ_EPI_RELU2) {
                s.x = fmaxf(s.x, 0.f); s.y = fmaxf(s.y, 0.f); s.z = fmaxf(s.z, 0.f); s.w = fmaxf(s.w, 0.f);
                s.x *= s.x; s.y *= s.y; s.z *= s.z; s.w *= s.w;
            } else if (a.epilogue == RWKVQ_EPI_ADD) {
                if (full) {
                    const float4 rv = __ldcg(reinterpret_cast<const float4*>(resid + o));
                    s.x = __fadd_rn(s.x, rv.x); s.y = __fadd_rn(s.y, rv.y); s.z = __fadd_rn(s.z, rv.z); s.w = __fadd_rn(s.w, rv.w);
                } else {
                    s.x = __fadd_rn(s.x, __ldcg(resid + o));
                    if (row + 1 < t.rows) s.y = __fadd_rn(s.y, __ldcg(resid + o + 1));
                    if (row + 2 < t.rows) s.z = __fadd_rn(s.z, __ldcg(resid + o + 2));
                    if (row + 3 < t.rows) s.w = __fadd_rn(s.w, __ldcg(resid + o + 3));
                }
            }
            if (full) {
                *reinterpret_cast<float4*>(y + o) = s;
            } else {
                y[o] = s.x;
                if (row + 1 < t.rows) y[o + 1] = s.y;
                if (row + 2 < t.rows) y[o + 2] = s.z;
                if (row + 3 < t.rows) y[o + 3] = s.w;
            }
            if (a.amax_out[blockIdx.y] != nullptr) {
                // |v| as int bits orders like the float; a NaN compares above every number and so survives
                float m = fabsf(s.x);
                if (row + 1 < t.rows) m = fmaxf(m, fabsf(s.y)) + 0.f * s.y;
                if (row + 2 < t.rows) m = fmaxf(m, fabsf(s.z)) + 0.f * s.z;
                if (row + 3 < t.rows) m = fmaxf(m, fabsf(s.w)) + 0.f * s.w;
                atomicMax(reinterpret_cast<int*>(s_omax) + n, __float_as_int(fabsf(m)));
            }
        }
    }
    tb_mark(a, 7);
    cluster.sync();          // nobody leaves while a peer still reads its partial tile
    tb_mark(a, 8);
    if (!failed && a.amax_out[blockIdx.y] != nullptr && tid < nn) {
        const int bits = reinterpret_cast<const int*>(s_omax)[tid];
        if (bits != 0) atomicMax(reinterpret_cast<int*>(a.amax_out[blockIdx.y]) + n0 + tid, bits);
    }
    if (warp == 0) tmem_dealloc(tmem, TM_COLS);
}

namespace {

template <int NT, bool EX>
int launch_tcb(TcbArgs& a, int n_mats, int n_groups, int row_tiles, cudaStream_t s) {
    // single-term: four slabs of weights and activations; two-term: two slabs of each of p, e, hi, lo + the min operands
    const size_t smem = 1024 + static_cast<size_t>(4) * (kGmRows * 128 + NT * 128) + (EX ? 2 * 16 * (kGmRows + NT) : 0);
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
    if (dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcb_kernel<NT, EX>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return fail(RWKVQ_E_LIMIT, "rwkvq_gemm_tcb: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        e = cudaFuncSetAttribute(gemm_tcb_kernel<NT, EX>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);      // clusters of 16
        if (e != cudaSuccess) return fail(RWKVQ_E_LIMIT, "rwkvq_gemm_tcb: cluster size attribute: %s", cudaGetErrorString(e));
        if (dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(row_tiles * a.ks, n_mats, n_groups);
    cfg.blockDim = dim3(kTbThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = a.ks; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_tcb_kernel<NT, EX>, a);
    if (le != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_gemm_tcb: %s", cudaGetErrorString(le));
    return RWKVQ_OK;
}

}  // namespace

int g_tcb_force_ks = 0;        // profiling aid (rwkvq_profiling.h): cluster size override

// RWKVQ_TCB=0 in the environment keeps the small-batch linears on the mma.sync kernel (A/B comparisons)
bool tcb_enabled() {
    static const bool on = [] { const char* e = getenv("RWKVQ_TCB"); return !(e && e[0] == '0'); }();
    return on && g_tcb_force_ks >= 0;          // rwkvq_profiling_tcb_force(-1) switches it off at run time
}
bool tcb_forced() { return g_tcb_force_ks > 0;
}

// Whether the tcgen05 small-batch kernel serves the tensor: sb6 / sym in the layouts the prefill
// kernel's producer reads (block 32 x 8 and 16 x 16), columns a multiple of 256.
bool gemm_tcb_ok(const rwkvq_qtensor& t) {
    if (t.cols % 256 != 0 || t.cols < 256) return false;
    if (t.kind == RWKVQ_KIND_SB6) return t.gs == 32 && t.sb == 8;
    if (t.kind == RWKVQ_KIND_SYM) return t.gs == 16 && t.sb == 16 && (t.bits == 8 || (t.qh && t.qh2));
    return false;
}

// Same contract as launch_gemv_batch (rwkvq_common.cuh), plus the device status word.  `exact`: the
// two-term kernel; with half_in its rows are scaled to at most 2^9 and it needs xs_lo[k] = fp16(x * 2^s
// - xs[k]) and xs_sum[k] (TcbArgs::xsum) beside xs[k].
int launch_gemm_tcb(const rwkvq_qtensor* ts, int n_mats, const void* const* xs, bool half_in, const float* const* scales,
                    int N, long long ldx, float* const* ys, long long ldy, int epilogue, const float* const* resids,
                    float* const* amax_outs, int* status, cudaStream_t s, bool exact, const void* const* xs_lo,
                    const void* const* xs_sum) {
    RWKVQ_REQUIRE(n_mats >= 1 && n_mats <= kTbMaxMats, RWKVQ_E_LIMIT, "rwkvq_gemm_tcb: %d matrices", n_mats);
    TcbArgs a{};
    for (int k = 0; k < n_mats; ++k) {
        RWKVQ_REQUIRE(gemm_tcb_ok(ts[k]) && ts[k].kind == ts[0].kind && ts[k].bits == ts[0].bits && ts[k].rows == ts[0].rows &&
                          ts[k].cols == ts[0].cols, RWKVQ_E_SHAPE, "rwkvq_gemm_tcb: fused matrices must share layout and shape");
        RWKVQ_REQUIRE(xs[k] && ys[k] && scales[k], RWKVQ_E_NULL, "rwkvq_gemm_tcb: x, its scales or y is null");
        RWKVQ_REQUIRE(aligned(xs[k], 16) && ldx % 8 == 0, RWKVQ_E_ALIGN, "rwkvq_gemm_tcb: x rows must be 16-byte aligned (ldx %% 8)");
        a.t[k] = make_view(ts[k]);
        if (half_in) { a.x16[k] = static_cast<const __half*>(xs[k]); a.unscale[k] = scales[k]; }
        else { a.x[k] = static_cast<const float*>(xs[k]); a.amax[k] = scales[k]; }
        if (half_in && exact) {
            RWKVQ_REQUIRE(xs_lo && xs_lo[k] && aligned(xs_lo[k], 16) && xs_sum && xs_sum[k] && aligned(xs_sum[k], 16), RWKVQ_E_NULL,
                          "rwkvq_gemm_tcb: the low halves or the block sums of x are missing");
            a.x16lo[k] = static_cast<const __half*>(xs_lo[k]);
            a.xsum[k] = static_cast<const __half*>(xs_sum[k]);
        }
        a.y[k] = ys[k]; a.resid[k] = resids ? resids[k] : nullptr;
        a.amax_out[k] = amax_outs ? amax_outs[k] : nullptr;
        RWKVQ_REQUIRE(epilogue != RWKVQ_EPI_ADD || a.resid[k], RWKVQ_E_NULL, "rwkvq_gemm_tcb: resid is null");
    }
    a.ldx = ldx; a.ldy = ldy; a.n_tokens = N; a.epilogue = epilogue; a.status = status;
    a.trace = g_batch_trace;
    const int rows = ts[0].rows, cols = ts[0].cols;
    const int nt = N <= 16 ? 16 : N <= 32 ? 32 : 64;
    const int n_groups = (N + nt - 1) / nt;
    const int row_tiles = (rows + kGmRows - 1) / kGmRows, n_sb = cols / kTbSbK;
    // cluster size: a divisor of the super-block count, at most 8; cost model in microseconds: waves of
    // resident CTAs (two per SM) x (set-up and first loads + super-blocks) + reduction
    const int tiles = row_tiles * n_mats * n_groups;
    int best_ks = 1;
    double best = 1e30;
    for (int c = 1; c <= 8; ++c) {
        if (n_sb % c) continue;
        const int waves = (tiles * c + 2 * 148 - 1) / (2 * 148);
        const double t = waves * (2.5 + (exact ? 1.8 : 0.9) * (n_sb / c)) + 2.0 + 0.15 * c;
        if (t < best) { best = t; best_ks = c; }
    }
    if (g_tcb_force_ks > 0 && n_sb % g_tcb_force_ks == 0 && g_tcb_force_ks <= 16) best_ks = g_tcb_force_ks;
    a.ks = best_ks;
    a.passes = n_sb / best_ks * (exact ? 2 : 1);
    if (exact) {
        switch (nt) {
            case 16: return launch_tcb<16, true>(a, n_mats, n_groups, row_tiles, s);
            case 32: return launch_tcb<32, true>(a, n_mats, n_groups, row_tiles, s);
            default: return launch_tcb<64, true>(a, n_mats, n_groups, row_tiles, s);
        }
    }
    switch (nt) {
        case 16: return launch_tcb<16, false>(a, n_mats, n_groups, row_tiles, s);
        case 32: return launch_tcb<32, false>(a, n_mats, n_groups, row_tiles, s);
        default: return launch_tcb<64, false>(a, n_mats, n_groups, row_tiles, s);
    }
}

}  // namespace rwkvq

extern "C" void rwkvq_profiling_tcb_force(int force_ks) { rwkvq::g_tcb_force_ks = force_ks; }
