// Single-vector decode GEMV on the integer tensor-core path: the stand-alone kernel,
// its launcher and the relayout kernels.  The arithmetic is described in rwkvq_gemv_mma.cuh.
#include <cstdlib>

#include "rwkvq_gemv_mma.cuh"

namespace rwkvq {


// Persistent kernel: gridDim.x CTAs walk the 16-row tiles of matrix blockIdx.y with
// stride gridDim.x * WT.  Inside a CTA step the 8 warps form WT tiles x WK slices
// of the K loop; the activations are prepared once per CTA.  Each warp sees a flat
// sequence of work items (tile, iteration); the loads of item n+1 are issued
// before item n is consumed.
// ZS: the exact zero-group skip (see prepare_x / load_frag), a compile-time variant so that launches
// without it carry none of its instructions
template <int L, int WK, bool SPLIT, bool ZS>      // SPLIT: the K loop is also split across gridDim.z CTAs
__global__ void __launch_bounds__(kMmaWarps * 32, 2) gemv_mma_kernel(const MmaArgs a) {
    using G = Geo<L>;
    constexpr int WT = kMmaWarps / WK;
    extern __shared__ __align__(16) unsigned char smem[];
    const QView& q = a.t[blockIdx.y];
    const int n_in = q.cols;
    int8_t* dig = reinterpret_cast<int8_t*>(smem);
    float* xs16 = reinterpret_cast<float*>(dig + 3 * n_in);
    float* red = xs16 + (n_in >> 4);                                     // [2][kMmaWarps * 16]
    uint8_t* zflag = reinterpret_cast<uint8_t*>(red + 2 * kMmaWarps * 16);   // [n_in / 32] all-zero groups of the activations

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int tl = warp / WK, ks = warp % WK;
    const int KS = SPLIT ? static_cast<int>(gridDim.z) : 1;  // K slices across CTAs
    const int n_iters = n_in / G::KI / KS;                  // iterations of this CTA's slice
    const int it0 = SPLIT ? blockIdx.z * n_iters : 0;
    const int n_tiles = (q.rows + 15) >> 4;
    const int step = gridDim.x * WT;
    const int ipt = (n_iters - ks + WK - 1) / WK;          // this warp's iterations per tile
    const int n_steps = ((n_tiles + WT - 1) / WT - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                        static_cast<int>(gridDim.x);
    const int n_items = n_steps * ipt;
    // prefetch side: item counter -> (tile, iteration)
    int i_n = 0, i_tile = blockIdx.x * WT + tl, i_j = 0;
    Frag<L> nxt;
    if (ZS) nxt = Frag<L>{};               // skipped loads leave the fragment as it was: start from zeros
    const uint8_t* zf = nullptr;           // set once the activations are prepared
    auto fetch_next = [&]() {
        if (i_n < n_items && i_tile < n_tiles) {
            const int r0 = min(i_tile * 16 + g, q.rows - 1), r1 = min(i_tile * 16 + g + 8, q.rows - 1);
            if (ZS) load_frag<L>(nxt, q, r0, r1, it0 + ks + i_j * WK, t, zf);
            else load_frag<L>(nxt, q, r0, r1, it0 + ks + i_j * WK, t);
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
    const float unscale = prepare_x(xv, a.x_dtype, n_in, x_bits<L>(), dig, xs16, red, finite, ZS ? zflag : nullptr);
    __syncthreads();
    // exact sparsity skip: groups of 32 columns whose activations are all zero (relu(k)^2 in the channel
    // mix) are not read from the second fetch on
    if (ZS) zf = zflag;

    int c_n = 0, buf = 0;
    for (int base = blockIdx.x * WT; base < n_tiles; base += step, buf ^= 1) {
        const int tile = base + tl;
        float acc0 = 0.f, acc1 = 0.f;     // rows g, g+8 of this tile
        for (int j = 0; j < ipt; ++j, ++c_n) {
            const Frag<L> cur = nxt;
            fetch_next();
            if (tile >= n_tiles) continue;
            const int it = it0 + ks + j * WK;

            consume_frag<L>(cur, it, g, t, dig, n_in, xs16, acc0, acc1);
        }
        // the 4 lanes of a quad hold the 8 blocks of each iteration
        acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 1); acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 2);
        acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 1); acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 2);
        float* rb = red + buf * (kMmaWarps * 16);
        if (t == 0) { rb[warp * 16 + g] = acc0; rb[warp * 16 + g + 8] = acc1; }
        __syncthreads();
        if (!SPLIT) {
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
    if (t.kind == RWKVQ_KIND_RTN && t.bits > 4 && t.cols % 128 == 0 && aligned(t.codes, 16)) return ML_RTN8;
    return -1;
}

int g_zero_skip = -1;                      // -1: read RWKVQ_ZERO_SKIP from the environment at first use
static bool zero_skip_enabled() {
    if (g_zero_skip < 0) {
        const char* e = getenv("RWKVQ_ZERO_SKIP");
        g_zero_skip = (e != nullptr && e[0] == '1') ? 1 : 0;
    }
    return g_zero_skip == 1;
}

constexpr int kResidentCtas = 2 * 148;     // 2 CTAs of 256 threads per SM at <= 128 registers
constexpr int kSplitMaxRows = 4096;        // rows a K-split launch may have (scratch sizing)
constexpr int kSplitMaxSlices = 4;

// Scratch of a K-split launch: partial sums, then the (self-resetting) arrival counters.
size_t gemv_mma_scratch_bytes() {
    return sizeof(float) * kSplitMaxSlices * kMmaMaxFused * kSplitMaxRows + sizeof(unsigned int) * 1024;
}

template <int L, int WK, bool SPLIT, bool ZS>
static int launch_one_zs(MmaArgs& a, int rows, int cols, int n_mats, int KS, cudaStream_t s) {
    constexpr int WT = kMmaWarps / WK;
    const size_t smem = 3 * static_cast<size_t>(cols) + 4 * (cols / 16) + 2 * kMmaWarps * 16 * 4 + ((cols / 32 + 15) / 16) * 16;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<L, WK, SPLIT, ZS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
        if (e != cudaSuccess) return fail(RWKVQ_E_LIMIT, "gemv_mma: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    const int units = ((rows + 15) / 16 + WT - 1) / WT;
    const int cap = kResidentCtas / (n_mats * KS) > 0 ? kResidentCtas / (n_mats * KS) : 1;
    a.rows_padded = ((rows + 15) / 16) * 16;
    cudaError_t le = launch_pdl(gemv_mma_kernel<L, WK, SPLIT, ZS>, dim3(units < cap ? units : cap, n_mats, KS),
                                dim3(kMmaWarps * 32), smem, s, a);
    if (le != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "gemv_mma: %s", cudaGetErrorString(le));
    return RWKVQ_OK;
}

template <int L, int WK, bool SPLIT = false>
static int launch_one(MmaArgs& a, int rows, int cols, int n_mats, int KS, cudaStream_t s) {
    // The zero-group skip is opt-in (RWKVQ_ZERO_SKIP=1): on this part a 16-byte hole saves no DRAM traffic
    // (whole 64-128-byte lines are fetched) and the variant costs ~0.2 us per launch.  When on: rows as long as
    // the channel-mix hidden vector, the one input with exact zeros, and the layouts whose loader can leave a
    // group unread.
    if (zero_skip_enabled() && cols >= 4096 && (L <= ML_SB6_6 || L == ML_SYM6))
        return launch_one_zs<L, WK, SPLIT, true>(a, rows, cols, n_mats, KS, s);
    return launch_one_zs<L, WK, SPLIT, false>(a, rows, cols, n_mats, KS, s);
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
    // the kernel gives every slice n_iters / KS iterations: only an exact division covers the row
    if (scratch && n_iters >= 16 && rows <= kSplitMaxRows) {
        if (tiles * n_mats * 4 <= kResidentCtas && n_iters >= 32 && n_iters % 4 == 0) KS = 4;
        else if (tiles * n_mats * 2 <= kResidentCtas && n_iters % 2 == 0) KS = 2;
    }
    if (KS > 1) {
        a.partial = scratch;
        a.counters = reinterpret_cast<unsigned int*>(scratch + kSplitMaxSlices * kMmaMaxFused * kSplitMaxRows);
        return launch_one<L, 8, true>(a, rows, cols, n_mats, KS, s);
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
        case ML_RTN8: return launch_wk<ML_RTN8>(a, rows, cols, n_mats, scratch, s);
        default: return launch_wk<ML_SYM8>(a, rows, cols, n_mats, scratch, s);
    }
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" void rwkvq_profiling_zero_skip(int on) { g_zero_skip = on < 0 ? -1 : (on ? 1 : 0); }

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
                  "rwkvq_gemv_static: needs an sb6 tensor with relayouted records/planes, a sym tensor or per-row int8");
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
