// Dequant-fused tensor-core GEMM for many right-hand sides (prefill, batched decode):
//     y[n, o] = epi( sum_c W[o, c] * x[n, c] ),   n < M tokens.
//
// tcgen05 formulation: the WEIGHTS are the M = 128 operand, the tokens are the UMMA N
// dimension (16..256), so the packed weight stream is read exactly once per token tile
// and the accumulator D[128 out-rows, N tokens] lives in tensor memory.
//   a pre-pass writes the activations once as fp16, scaled per token by a power of two so
//     that no value leaves the fp16 range;
//   producers (16 warps = 512 threads; two more warps hold the TMA and the MMA issuer lanes): unpack a [128 rows, 64 K] slab of the file
//     layout (nibbles / planes / int8 + block scales) to fp16 = fp16(q*s + m) with one
//     HFMA2 per two weights (s and m ARE fp16 values by the codec's definition, so the
//     fused multiply-add rounds the exact value once) and store it K-major with the
//     128-byte swizzle the UMMA shared-memory descriptor expects; the packed bytes of the
//     next slab are already in flight (register prefetch);
//   the activation slab [N, 64 K] of each stage arrives by TMA (cp.async.bulk.tensor.2d,
//     SWIZZLE_128B, mbarrier complete_tx), issued by one thread one stage ahead; rows
//     beyond M are zero-filled by the tensor map;
//   one elected thread issues four tcgen05.mma (K = 16 each) per slab and commits them
//     to the mbarrier that frees the slab's ring stage;
//   epilogue: tcgen05.ld of the accumulator (lane = output row, column = token),
//     un-scale, relu^2 / residual, coalesced stores.
// Every wait on an mbarrier is bounded; on expiry the kernel records an error code,
// skips the remaining work, frees its tensor memory and returns.
#include "rwkvq_tc.cuh"

namespace rwkvq {

constexpr int kGmProducers = 512;     // warps 0-15 unpack weights (and run the epilogue)
constexpr int kGmThreads = 576;       // + warp 16: one lane issues the MMAs; warp 17: one lane issues the TMA loads
constexpr int kGmMaxBSlots = 8;       // activation slabs in flight (TMA)
// activation slab slots: as many pairs as fit beside the two weight stages
__host__ __device__ constexpr int gemm_b_slots(int nt, int km, int rh = 1) {
    return rh == 2 ? 3 : nt >= 256 ? 4 : (nt >= 128 && km == 256) ? 6 : 8;
}

struct GemmArgs {
    QView t;
    const float* x;        // [M, ldx] fp32 (read by the pre-pass only)
    long long ldx;
    float* y;              // [M, ldy] fp32
    long long ldy;
    const float* resid;
    const float* row_scale;   // [M] power of two: x * row_scale fits fp16
    int* status;              // device word: first error code, 0 = ok
    unsigned int* counters;   // [row tiles * token tiles] arrivals of the K slices (zeroed per call)
    float* partial;           // [CTA][NT][128] accumulator tiles of a K-split launch
    int M, epilogue;
    // optional timeline of CTA (0,0,0), nanoseconds of the global timer: [0] start, [1] accumulator
    // complete, [2] end; [8 + 4 i + {0 weights of macro-iteration i converted, 1 its stage was free,
    // 2 issuer saw it full, 3 issuer issued its MMAs}]
    unsigned long long* trace;
};

__device__ __forceinline__ void trace_mark(const GemmArgs& a, int slot) {
    if (a.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && slot < 512) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        a.trace[slot] = t;
    }
}

// Warps 0-15: producers (and the epilogue).  Warp 16, one lane: issues the MMAs.  Warp 17, one
// lane: issues the activation TMA loads.  Producers and issuer meet only through mbarriers:
//   bar_afull[s]  one arrival per producer warp (after every lane's proxy fence): the A slabs of stage s are written
//   bar_afree[s]  tcgen05.commit: the MMAs that read stage s have completed
//   bar_bfull[k]  TMA bytes of activation slot k have landed;  bar_bfree[k]  its MMAs completed
// NT = tokens per CTA tile (UMMA N): 16 .. 256;  KM = K of a macro-iteration: 256 (one super-block,
// four slabs) or 128 (two slabs; leaves room for the activation tiles of NT = 256);  RH = 128-row
// halves of the CTA's output tile: with RH = 2 every activation slab feeds two accumulators (all
// 512 tensor-memory columns at NT = 256), which halves the L2 -> SM traffic per FLOP, the bound
// of the one-accumulator form at large M.  The activation ring then holds three single slabs
// instead of two pairs (shared memory: 128 KB of weights + 96 KB of activations).  Measured: a
// deeper ring (K = 64 stages, five slabs) is no faster; the tensor pipe then runs at ~45 % because
// the shared memory itself is busy: per K = 64 the MMAs read 96 KB while 64 KB are written.
template <int NT, int KM, int RH>
__global__ void __launch_bounds__(kGmThreads, 1) gemm_tc_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap xmap) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int SLAB_BYTES = kGmRows * 128, B_BYTES = NT * 128;
    constexpr int kGmSlabs = KM / kGmK;                         // slabs per macro-iteration
    constexpr int kItems = KM / 32;                             // items (32 weights) per row and macro-iteration
    constexpr int kGmPasses = kGmRows * RH * kItems / kGmProducers;  // items per producer thread and macro-iteration
    constexpr int SPB = RH == 2 ? 1 : 2;                        // activation slabs per ring slot (one mbarrier each)
    constexpr int BS = gemm_b_slots(NT, KM, RH);
    constexpr uint32_t TM_COLS = RH * NT < 32 ? 32 : RH * NT;
    unsigned char* a_ring = smem;                                        // [2 stages][RH][slabs][SLAB_BYTES]
    unsigned char* b_ring = smem + 2 * RH * kGmSlabs * SLAB_BYTES;       // [BS][B_BYTES]
    __shared__ uint64_t bar_afull[2], bar_afree[2], bar_bfull[kGmMaxBSlots], bar_bfree[kGmMaxBSlots], bar_done;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_fail;
    __shared__ float s_unscale[NT];              // 1 / token scale (exact: the scales are powers of two)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const QView& t = a.t;
    const int row0 = blockIdx.x * kGmRows * RH, tok0 = blockIdx.y * NT;
    const int KS = gridDim.z;
    const int n_m = (t.cols / KM) / KS;                         // macro-iterations of this CTA's K slice
    const int m_first = blockIdx.z * n_m;                       // first macro-iteration, in units of KM

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) { mbar_init(&bar_afull[s], kGmProducers / 32); mbar_init(&bar_afree[s], 1); }
        for (int s = 0; s < BS; ++s) { mbar_init(&bar_bfull[s], 1); mbar_init(&bar_bfree[s], 1); }
        mbar_init(&bar_done, 1);
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Launched programmatically behind the pre-pass: everything up to the first use of the
    // activations (barrier set-up, TMEM, the first packed weights) overlaps with it.
    pdl_launch_dependents();
    if (warp == 0) tmem_alloc(&s_tmem, TM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    if (tid == 0) trace_mark(a, 0);

    constexpr int NP = BS / SPB;                                // slots of the activation ring
    const int n_pairs = n_m * kGmSlabs / SPB;                   // slot fills of this CTA
    if (warp == kGmProducers / 32 + 1) {
        // ------------------------------------------------------------------ activation loader
        // Activation slabs travel in groups of SPB (one mbarrier per group): slabs SPB q .. of this CTA
        // go to slot q % NP as soon as the MMAs that read its previous content have completed.
        if (lane == 0) {
            pdl_wait();                                         // the fp16 activations come from the pre-pass
            int ps = 0, round = 0;
            for (int q = 0; q < n_pairs; ++q) {
                if (round > 0 && !mbar_wait_bounded(&bar_bfree[ps], (round - 1) & 1)) { s_fail = 1; break; }
                if (s_fail) break;
                mbar_expect_tx(&bar_bfull[ps], SPB * B_BYTES);
#pragma unroll
                for (int s2 = 0; s2 < SPB; ++s2)
                    tma_load_2d(b_ring + (SPB * ps + s2) * B_BYTES, &xmap, (m_first * kGmSlabs + SPB * q + s2) * kGmK, tok0,
                                &bar_bfull[ps]);
                if (++ps == NP) { ps = 0; ++round; }
            }
        }
    } else if (warp == kGmProducers / 32) {
        // ------------------------------------------------------------------ MMA issuer
        // A single thread executes dependent scalar code at a few cycles per instruction, so this
        // loop carries nothing but the waits, the MMAs and the commits: descriptors are formed by
        // adding slab offsets to two base descriptors.
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(NT);
            const uint64_t a_desc0 = umma_desc(smem_addr(a_ring)), b_desc0 = umma_desc(smem_addr(b_ring));
            constexpr int PPM = kGmSlabs / SPB;                  // slot fills per macro-iteration
            bool ok = true;
            int i = 0, pq = 0, ps = 0, bphase = 0;               // macro-iteration, pair in it, pair slot, slot phase
            for (int q = 0; q < n_pairs && ok; ++q) {
                const int st = i & 1;
                if (pq == 0) {
                    if (!mbar_wait_bounded(&bar_afull[st], (i >> 1) & 1)) { ok = false; break; }
                    trace_mark(a, 8 + 4 * i + 2);
                }
                if (!mbar_wait_bounded(&bar_bfull[ps], bphase)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int s2 = 0; s2 < SPB; ++s2) {
                    const uint64_t bd = b_desc0 + (static_cast<uint64_t>((SPB * ps + s2) * B_BYTES) >> 4);
#pragma unroll
                    for (int rh = 0; rh < RH; ++rh) {          // one accumulator per 128-row half
                        const uint64_t ad = a_desc0 + (static_cast<uint64_t>(((st * RH + rh) * kGmSlabs + pq * SPB + s2) * SLAB_BYTES) >> 4);
#pragma unroll
                        for (int k = 0; k < kGmK / 16; ++k)    // 32 bytes further along K per step
                            umma_f16(tmem + rh * NT, ad + 2 * k, bd + 2 * k, idesc, (q | s2 | k) ? 1u : 0u);
                    }
                }
                umma_commit(&bar_bfree[ps]);
                if (pq == PPM - 1) { umma_commit(&bar_afree[st]); trace_mark(a, 8 + 4 * i + 3); }
                if (++pq == PPM) { pq = 0; ++i; }
                if (++ps == NP) { ps = 0; bphase ^= 1; }
            }
            if (ok) umma_commit(&bar_done);
            else s_fail = 1;
        }
    } else {
        // ------------------------------------------------------------------ producers
        constexpr int PR = kGmProducers / kItems;               // rows per pass
        const int pit = tid % kItems, prow = tid / kItems;      // item of the macro-iteration, row within a pass
        Packed P0[kGmPasses], P1[kGmPasses];                    // packed bytes of macro-iterations i, i + 1 (static roles)
        auto load_all = [&](Packed (&P)[kGmPasses], int i) {
#pragma unroll
            for (int q = 0; q < kGmPasses; ++q)
                load_packed(P[q], t, min(row0 + PR * q + prow, t.rows - 1), ((m_first + i) * KM) >> 8,
                            (((m_first + i) * KM) >> 5 & 7) + pit);
        };
        auto produce = [&](Packed (&P)[kGmPasses], int i) {
            const int st = i & 1;
            // one lane per warp polls: 256 threads spinning on a shared-memory barrier starve the
            // issuer's own barrier, TMA and MMA instructions
            if (i >= 2) {
                if (lane == 0 && !s_fail && !mbar_wait_bounded(&bar_afree[st], ((i >> 1) - 1) & 1)) s_fail = 1;
                __syncwarp();
            }
            if (tid == 0) trace_mark(a, 8 + 4 * i + 1);
            if (!s_fail) {
#pragma unroll
                for (int q = 0; q < kGmPasses; ++q) {
                    const int r = PR * q + prow;                // row of the CTA's tile: half r / 128, row r % 128 of its slabs
                    unsigned char* slab = a_ring + ((st * RH + r / kGmRows) * kGmSlabs + (pit >> 1)) * SLAB_BYTES;
                    convert_store(P[q], t, r % kGmRows, (((m_first + i) * KM) >> 5 & 7) + pit, pit & 1, slab);
                }
            }
            fence_async_smem();                                 // generic-proxy stores -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_afull[st]);         // one arrival per warp: 512 arrivals on one word serialise
            if (tid == 0) trace_mark(a, 8 + 4 * i);
            if (i + 2 < n_m) load_all(P, i + 2);                // the registers are free again: two iterations ahead
        };
        load_all(P0, 0);
        if (n_m > 1) load_all(P1, 1);
        for (int i = 0; i < n_m; i += 2) {
            produce(P0, i);
            if (i + 1 < n_m) produce(P1, i + 1);
        }
    }
    // ---------------------------------------------------------------------- epilogue
    if (lane == 0 && !s_fail && !mbar_wait_bounded(&bar_done, 0)) s_fail = 1;
    __syncwarp();
    pdl_wait();                                                 // token scales, residual, K-split scratch
    if (tid < NT) s_unscale[tid] = (tok0 + tid < a.M) ? 1.0f / __ldcg(a.row_scale + tok0 + tid) : 0.f;
    tc_fence_after();
    __syncthreads();
    if (tid == 0) trace_mark(a, 1);
    if (s_fail) {
        if (tid == 0) atomicCAS(a.status, 0, RWKVQ_E_TIMEOUT);
    } else if (warp < kGmProducers / 32) {
        // warp w reads lanes 32*(w%4) .. +31 (= output rows); the warps that share a lane group split the tokens
        const int rl = (warp & 3) * 32 + lane;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        auto finish = [&](float r, int tok, int row) {
            if (tok < a.M && row < t.rows) {
                r = r * s_unscale[tok - tok0];
                const long long idx = tok * a.ldy + row;
                if (a.epilogue == RWKVQ_EPI_RELU2) { r = fmaxf(r, 0.f); r = r * r; }
                else if (a.epilogue == RWKVQ_EPI_ADD) r = __fadd_rn(r, __ldcg(a.resid + idx));
                a.y[idx] = r;
            }
        };
        if (KS == 1) {
#pragma unroll
            for (int rh = 0; rh < RH; ++rh)
                for (int c0 = (warp >> 2) * 8; c0 < NT; c0 += kGmProducers / 16) {
                    float v[8];
                    tmem_ld8(lane_base + rh * NT + c0, v);
#pragma unroll
                    for (int j = 0; j < 8; ++j) finish(v[j], tok0 + c0 + j, row0 + rh * kGmRows + rl);
                }
        } else {
            // this CTA's accumulator tile goes to its scratch slot [token][row]
            const size_t tile_id = static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x;
            float* mine = a.partial + (tile_id * KS + blockIdx.z) * (NT * kGmRows * RH);
#pragma unroll
            for (int rh = 0; rh < RH; ++rh)
                for (int c0 = (warp >> 2) * 8; c0 < NT; c0 += kGmProducers / 16) {
                    float v[8];
                    tmem_ld8(lane_base + rh * NT + c0, v);
#pragma unroll
                    for (int j = 0; j < 8; ++j) __stcg(mine + (c0 + j) * (kGmRows * RH) + rh * kGmRows + rl, v[j]);
                }
            __threadfence();
        }
    }
    if (KS > 1 && !s_fail) {                        // block-uniform: every thread takes the same path
        __shared__ unsigned int s_last;
        const size_t tile_id = static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x;
        __syncthreads();
        if (tid == 0) s_last = (atomicAdd(a.counters + tile_id, 1u) == static_cast<unsigned int>(KS - 1));
        __syncthreads();
        if (s_last && warp < kGmProducers / 32) {   // last K slice to arrive adds the tiles in slice order
            __threadfence();
            const float* base = a.partial + tile_id * KS * (NT * kGmRows * RH);
            // warps of one lane group take alternate groups of 8 tokens; 8 x 4 loads are in flight per
            // thread and every token's slices are added in slice order
#pragma unroll
            for (int rh = 0; rh < RH; ++rh)
            for (int c0 = (warp >> 2) * 8; c0 < NT; c0 += kGmProducers / 16) {
                const int rl = rh * kGmRows + (warp & 3) * 32 + lane, row = row0 + rl;
                float r[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) r[j] = 0.f;
                for (int z0 = 0; z0 < KS; z0 += 4) {
                    float pv[4][8];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            pv[u][j] = z0 + u < KS
                                           ? __ldcg(base + (static_cast<size_t>(z0 + u) * NT + c0 + j) * (kGmRows * RH) + rl)
                                           : 0.f;
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int j = 0; j < 8; ++j) r[j] += pv[u][j];
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int tok = tok0 + c0 + j;
                    if (tok < a.M && row < t.rows) {
                        float v = r[j] * s_unscale[tok - tok0];
                        const long long idx = tok * a.ldy + row;
                        if (a.epilogue == RWKVQ_EPI_RELU2) { v = fmaxf(v, 0.f); v = v * v; }
                        else if (a.epilogue == RWKVQ_EPI_ADD) v = __fadd_rn(v, __ldcg(a.resid + idx));
                        a.y[idx] = v;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0) trace_mark(a, 2);
    if (warp == 0) tmem_dealloc(tmem, TM_COLS);
}

// Pre-pass, one CTA per token: power-of-two scale so that |x * scale| <= 2^14, and the
// scaled row as fp16 (the tensor the TMA loads read).
__global__ void __launch_bounds__(256) row_scale_kernel(const float* x, long long ldx, int cols, float* scale,
                                                        __half* x16, long long pitch, uint4* header, int header_words16) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();                 // x comes from the previous kernel, which may also still read this workspace
    if (blockIdx.x == 0)        // status word and K-split arrival counters of the GEMM that follows
        for (int i = threadIdx.x; i < header_words16; i += 256) header[i] = make_uint4(0, 0, 0, 0);
    const float* row = x + blockIdx.x * ldx;
    float amax = 0.f;
    for (int i = threadIdx.x; i < cols; i += 256) amax = fmaxf(amax, fabsf(__ldcg(row + i)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
    int e = 0;
    if (amax > 0.f && amax < INFINITY) frexpf(amax, &e);
    const float sc = ldexpf(1.f, 14 - e);
    if (threadIdx.x == 0) scale[blockIdx.x] = sc;
    __half2* out = reinterpret_cast<__half2*>(x16 + static_cast<size_t>(blockIdx.x) * pitch);
    for (int i = threadIdx.x; i < (cols >> 1); i += 256) {
        const float2 v = __ldcg(reinterpret_cast<const float2*>(row) + i);
        out[i] = __floats2half2_rn(v.x * sc, v.y * sc);
    }
}

// For activations that arrive already scaled (rwkvq_gemm_x16): only the header is zeroed.
__global__ void __launch_bounds__(256) gemm_header_zero_kernel(uint4* header, int header_words16) {
    pdl_launch_dependents();
    pdl_wait();                 // the previous kernel may still read this workspace
    for (int i = threadIdx.x; i < header_words16; i += 256) header[i] = make_uint4(0, 0, 0, 0);
}

}  // namespace rwkvq

using namespace rwkvq;

namespace {
unsigned long long* g_gemm_trace = nullptr;      // set by rwkvq_profiling_gemm_trace (rwkvq_profiling.h)
int g_gemm_acc_mode = 0;                         // rwkvq_profiling_gemm_acc_mode: 0 launcher's choice, 1 never / 2 always 256-row tiles
constexpr int kGemmResident = 2 * 148;     // accumulator tiles the K-split scratch holds
constexpr int kGemmSms = 148;
// Row pitch of the fp16 activation copy: 128 bytes more than the row, so that the 128 rows
// of a TMA box do not all map to the same L2 slice (a power-of-two pitch does).
inline size_t x16_pitch(int cols) { return static_cast<size_t>(cols) + 64; }
constexpr size_t kGemmHeader = 8192;        // status word + arrival counters (zeroed every call)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// fp16 activations [M, cols] row-major; box = [NT tokens, 64 columns], 128-byte swizzle, zero fill
int make_xmap(CUtensorMap* map, const __half* x16, int M, int cols, int nt) {
    EncodeTiledFn enc = encode_tiled();
    RWKVQ_REQUIRE(enc != nullptr, RWKVQ_E_ARCH, "rwkvq_gemm: cuTensorMapEncodeTiled is not available");
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(x16_pitch(cols)) * sizeof(__half)};
    const cuuint32_t box[2] = {kGmK, static_cast<cuuint32_t>(nt)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(x16), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    RWKVQ_REQUIRE(r == CUDA_SUCCESS, RWKVQ_E_LAUNCH, "rwkvq_gemm: cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    return RWKVQ_OK;
}

template <int NT, int KM, int RH = 1>
int launch_gemm(GemmArgs& a, int rows, int cols, int M, float* partial, const __half* x16, cudaStream_t s) {
    CUtensorMap xmap;
    int mrc = make_xmap(&xmap, x16, M, cols, NT);
    if (mrc) return mrc;
    const size_t smem = static_cast<size_t>(2 * RH * (KM / kGmK)) * kGmRows * 128 + static_cast<size_t>(gemm_b_slots(NT, KM, RH)) * NT * 128 + 1024;
    // the attribute belongs to the (function, device) pair: remember it per device of this process
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
    if (dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<NT, KM, RH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
        if (e != cudaSuccess) return fail(RWKVQ_E_LIMIT, "rwkvq_gemm: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        if (dev < 64) configured[dev] = true;
    }
    const int rt = (rows + kGmRows * RH - 1) / (kGmRows * RH), tt = (M + NT - 1) / NT, n_m = cols / KM;
    // K slices across CTAs while the grid is below one CTA per SM (power of two, >= 2 super-blocks each)
    int KS = 1;
    while (rt * tt * KS < kGemmSms && n_m % (KS * 2) == 0 && n_m / (KS * 2) >= 2 && rt * tt * KS * 2 * RH <= kGemmResident &&
           rt * tt <= static_cast<int>((kGemmHeader - 256) / sizeof(unsigned int)))
        KS *= 2;
    a.partial = partial;
    cudaError_t le = launch_pdl(gemm_tc_kernel<NT, KM, RH>, dim3(rt, tt, KS), dim3(kGmThreads), smem, s, a, xmap);
    if (le != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_gemm: %s", cudaGetErrorString(le));
    return RWKVQ_OK;
}
int dispatch_gemm(GemmArgs& a, const rwkvq_qtensor* t, int M, float* partial, const __half* x16, cudaStream_t s) {
    if (M <= 16) return launch_gemm<16, 256>(a, t->rows, t->cols, M, partial, x16, s);
    if (M <= 32) return launch_gemm<32, 256>(a, t->rows, t->cols, M, partial, x16, s);
    if (M <= 64) return launch_gemm<64, 256>(a, t->rows, t->cols, M, partial, x16, s);
    // 256-token tiles (every converted weight serves 256 tokens) once they still give the
    // SMs enough CTAs or a long K loop; otherwise 128-token tiles
    const int tiles256 = ((t->rows + kGmRows - 1) / kGmRows) * ((M + 255) / 256);
    // 256 rows per CTA (two accumulators per activation slab) once such tiles alone fill the SMs and
    // their last, partly filled wave does not cost more than the form gains (kTwoAccGain, measured)
    const int tiles2 = (t->rows / (2 * kGmRows)) * ((M + 255) / 256);
    auto wave_eff = [](int tiles) { return static_cast<double>(tiles) / (((tiles + kGemmSms - 1) / kGemmSms) * kGemmSms); };
    constexpr double kTwoAccGain = 1.08;
    const bool two_pays = tiles2 >= kGemmSms && wave_eff(tiles2) * kTwoAccGain >= wave_eff(tiles256);
    if (M > 128 && t->rows % (2 * kGmRows) == 0 && g_gemm_acc_mode != 1 && (two_pays || g_gemm_acc_mode == 2))
        return launch_gemm<256, 128, 2>(a, t->rows, t->cols, M, partial, x16, s);
    if (M > 128 && (tiles256 >= 64 || t->cols >= 4096))
        return launch_gemm<256, 128>(a, t->rows, t->cols, M, partial, x16, s);
    return launch_gemm<128, 256>(a, t->rows, t->cols, M, partial, x16, s);
}
}  // namespace

extern "C" {

// header | row scales [M] | K-split accumulator tiles (one wave of CTAs x 128 x NT floats) | fp16 activations
static size_t gemm_ws_partial_off(size_t m) { return kGemmHeader + ((sizeof(float) * m + 255) / 256) * 256; }
static size_t gemm_ws_x16_off(size_t m) {
    const size_t nt = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : m <= 128 ? 128 : 256;
    return gemm_ws_partial_off(m) + sizeof(float) * kGemmResident * kGmRows * nt;
}
size_t rwkvq_gemm_workspace_bytes_for(int M, int max_cols) {
    const size_t m = static_cast<size_t>(M < 1 ? 1 : M);
    return gemm_ws_x16_off(m) + sizeof(__half) * m * (static_cast<size_t>(max_cols) + 64) + 256;
}
void rwkvq_profiling_gemm_trace(void* buf512) { g_gemm_trace = static_cast<unsigned long long*>(buf512); }
void rwkvq_profiling_gemm_acc_mode(int mode) { g_gemm_acc_mode = mode; }

size_t rwkvq_gemm_workspace_bytes(int M) { return rwkvq_gemm_workspace_bytes_for(M, 16384); }

int rwkvq_gemm(const rwkvq_qtensor* t, const float* x, int M, int64_t ldx, float* y, int64_t ldy, int epilogue,
               const float* resid, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = validate_qtensor(t, "rwkvq_gemm");
    if (rc) return rc;
    RWKVQ_REQUIRE(t->kind == RWKVQ_KIND_SB6 || t->kind == RWKVQ_KIND_SYM, RWKVQ_E_DTYPE,
                  "rwkvq_gemm: only sb6 and sym tensors have a tensor-core path (kind %d)", t->kind);
    RWKVQ_REQUIRE(x && y && workspace, RWKVQ_E_NULL, "rwkvq_gemm: null pointer");
    RWKVQ_REQUIRE(M >= 1 && ldx >= t->cols && ldy >= t->rows, RWKVQ_E_SHAPE, "rwkvq_gemm: M=%d ldx=%lld ldy=%lld", M,
                  (long long)ldx, (long long)ldy);
    RWKVQ_REQUIRE(aligned(x, 16) && ldx % 4 == 0 && aligned(workspace, 256), RWKVQ_E_ALIGN,
                  "rwkvq_gemm: x and its row stride must be 16-byte aligned, the workspace 256-byte aligned");
    RWKVQ_REQUIRE(workspace_bytes >= rwkvq_gemm_workspace_bytes_for(M, t->cols), RWKVQ_E_LIMIT,
                  "rwkvq_gemm: workspace %zu < %zu bytes", workspace_bytes, rwkvq_gemm_workspace_bytes_for(M, t->cols));
    RWKVQ_REQUIRE(epilogue >= RWKVQ_EPI_NONE && epilogue <= RWKVQ_EPI_ADD, RWKVQ_E_DTYPE, "rwkvq_gemm: epilogue %d", epilogue);
    RWKVQ_REQUIRE(epilogue != RWKVQ_EPI_ADD || resid, RWKVQ_E_NULL, "rwkvq_gemm: resid is null");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    char* ws = static_cast<char*>(workspace);
    GemmArgs a{};
    a.t = make_view(*t);
    a.x = x; a.ldx = ldx; a.y = y; a.ldy = ldy; a.resid = resid; a.M = M; a.epilogue = epilogue;
    a.status = reinterpret_cast<int*>(ws);
    a.counters = reinterpret_cast<unsigned int*>(ws + 256);
    float* scale = reinterpret_cast<float*>(ws + kGemmHeader);
    float* partial = reinterpret_cast<float*>(ws + gemm_ws_partial_off(M));
    __half* x16 = reinterpret_cast<__half*>(ws + gemm_ws_x16_off(M));
    a.row_scale = scale;
    a.trace = g_gemm_trace;
    cudaError_t le = launch_pdl(row_scale_kernel, dim3(M), dim3(256), 0, s, x, static_cast<long long>(ldx), t->cols, scale, x16,
                                static_cast<long long>(x16_pitch(t->cols)), reinterpret_cast<uint4*>(ws),
                                static_cast<int>(kGemmHeader / 16));
    if (le != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_gemm(pre-pass): %s", cudaGetErrorString(le));
    rc = dispatch_gemm(a, t, M, partial, x16, s);
    if (rc) return rc;
    return check_launch("rwkvq_gemm");
}

size_t rwkvq_gemm_x16_pitch(int cols) { return x16_pitch(cols); }

int rwkvq_gemm_x16(const rwkvq_qtensor* t, const void* x16, const float* row_scale, int M, float* y, int64_t ldy,
                   int epilogue, const float* resid, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = validate_qtensor(t, "rwkvq_gemm_x16");
    if (rc) return rc;
    RWKVQ_REQUIRE(t->kind == RWKVQ_KIND_SB6 || t->kind == RWKVQ_KIND_SYM, RWKVQ_E_DTYPE,
                  "rwkvq_gemm_x16: only sb6 and sym tensors have a tensor-core path (kind %d)", t->kind);
    RWKVQ_REQUIRE(x16 && row_scale && y && workspace, RWKVQ_E_NULL, "rwkvq_gemm_x16: null pointer");
    RWKVQ_REQUIRE(M >= 1 && ldy >= t->rows, RWKVQ_E_SHAPE, "rwkvq_gemm_x16: M=%d ldy=%lld", M, (long long)ldy);
    RWKVQ_REQUIRE(aligned(x16, 16) && aligned(workspace, 256), RWKVQ_E_ALIGN,
                  "rwkvq_gemm_x16: x16 must be 16-byte aligned, the workspace 256-byte aligned");
    RWKVQ_REQUIRE(workspace_bytes >= gemm_ws_x16_off(M), RWKVQ_E_LIMIT, "rwkvq_gemm_x16: workspace %zu < %zu bytes",
                  workspace_bytes, gemm_ws_x16_off(M));
    RWKVQ_REQUIRE(epilogue >= RWKVQ_EPI_NONE && epilogue <= RWKVQ_EPI_ADD, RWKVQ_E_DTYPE, "rwkvq_gemm_x16: epilogue %d", epilogue);
    RWKVQ_REQUIRE(epilogue != RWKVQ_EPI_ADD || resid, RWKVQ_E_NULL, "rwkvq_gemm_x16: resid is null");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    char* ws = static_cast<char*>(workspace);
    GemmArgs a{};
    a.t = make_view(*t);
    a.y = y; a.ldy = ldy; a.resid = resid; a.M = M; a.epilogue = epilogue;
    a.status = reinterpret_cast<int*>(ws);
    a.counters = reinterpret_cast<unsigned int*>(ws + 256);
    a.row_scale = row_scale;
    a.trace = g_gemm_trace;
    cudaError_t le = launch_pdl(gemm_header_zero_kernel, dim3(1), dim3(256), 0, s, reinterpret_cast<uint4*>(ws),
                                static_cast<int>(kGemmHeader / 16));
    if (le != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_gemm_x16(header): %s", cudaGetErrorString(le));
    rc = dispatch_gemm(a, t, M, reinterpret_cast<float*>(ws + gemm_ws_partial_off(M)), static_cast<const __half*>(x16), s);
    if (rc) return rc;
    return check_launch("rwkvq_gemm_x16");
}

}  // extern "C"
