// The four LoRA branches of the time-mix block for a BATCH of decode streams on the tensor
// cores (backends/metal/quant_model.py:462-526: y_br = act_br(x_br @ W1_br) @ W2_br with
// act = tanh / none / sigmoid / none for the decay, in-context rate, gate and value-residual
// branches).  The per-stream kernels of rwkvq_decode.cu serve up to 8 streams; beyond that
// they re-read the matrices for every group of 8 streams and run on the SIMT pipes.  Here:
//
//   down   grid (8 K slices = one cluster, branch x stream group, 32-column groups of the rank):
//          a CTA turns its [K/8, 32] slice of W1 (file bytes, stored [in, out]) into fp16 in the
//          loader's precision fp16(bf16(.)), which is exact, and its slice of the activations
//          into an fp16 pair hi + lo (x to ~2^-22), multiplies on mma.sync.m16n8k16 with the
//          streams as the 16-row operand and fp32 accumulation, and the 8 slices of a cluster are
//          added in rank order through distributed shared memory; the activation function is
//          applied there and h [streams, rank] is written once.
//   up     grid (32-column tiles of D, branch x stream group): h as an fp16 pair times the
//          [rank, 32] slice of W2, no split of the short K = rank.
// Both launches are programmatic-dependent; the weights are staged before the producer's
// results are awaited.  No wait spins: the only cross-CTA synchronisation is the hardware
// cluster barrier.
#include <cooperative_groups.h>

#include <algorithm>

#include "rwkvq_decode_parts.cuh"

namespace cg = cooperative_groups;

namespace rwkvq {

constexpr int kLmmThreads = 256;
constexpr int kLmmSlices = 8;            // K slices of the down projection = cluster size
constexpr int kLmmRC = 32;               // rank columns per CTA of the down projection
constexpr int kLmmUpCols = 32;           // output columns per CTA of the up projection
constexpr int kLmmPad = 8;               // halves of padding per shared-memory row (bank spread)
constexpr int kLmmMaxSmem = 200 * 1024;

struct LoraMmaArgs {
    QView t1[4], t2[4];
    const float* x[4];       // [N, ldx] per branch
    float* h;                // [4][n_stride][max_rank] activations of the rank space
    float* y[4];             // [N, ldy]
    int act[4];
    long long ldx, ldy;
    int n_tokens, n_stride, max_rank, n_br, D;
    int n_groups;            // stream groups of MT * 16; a CTA walks groups blockIdx.y / n_br, + gridDim.y / n_br, ...
};

__device__ __forceinline__ void lmm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// fp32 -> (hi, lo) fp16 with hi + lo = x to ~2^-22 relative
__device__ __forceinline__ void split4(const float4& v, uint2& hi, uint2& lo) {
    const __half2 h01 = __floats2half2_rn(v.x, v.y), h23 = __floats2half2_rn(v.z, v.w);
    const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
    const __half2 l01 = __floats2half2_rn(v.x - f01.x, v.y - f01.y), l23 = __floats2half2_rn(v.z - f23.x, v.w - f23.y);
    hi = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
    lo = make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
}

// rows [k0, k0 + kc) x columns [c0, c0 + nc) of a tensor stored [in, out] -> wk[row][col] fp16, the stored
// orientation (columns contiguous: coalesced loads, 8-byte conflict-free stores); the MMA's "col" operand is
// read from it with ldmatrix.trans.  nc is a multiple of 4.
__device__ __forceinline__ uint2 pack4h(const float (&w)[4]) {
    const __half2 a = __floats2half2_rn(w[0], w[1]), b = __floats2half2_rn(w[2], w[3]);      // exact: fp16 values
    return make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}
template <int MODE>
__device__ __forceinline__ void stage_wt(const QView& t, int k0, int kc, int c0, int nc, __half* wk, int pitch) {
    const int groups = nc >> 2;
    const int nb = MODE == 0 ? (t.cols + t.gs - 1) / t.gs : 0;
    const int total = kc * groups;
    if (MODE == 2) {
        for (int item = threadIdx.x; item < total; item += kLmmThreads) {
            const int k = item / groups, cg4 = item - k * groups;
            float w[4];
            lora_w4<2>(t, k0 + k, c0 + cg4 * 4, 0, 0, w);
            *reinterpret_cast<uint2*>(wk + k * pitch + cg4 * 4) = pack4h(w);
        }
        return;
    }
    // 8 items per thread with all their loads issued together (one item is a latency chain)
    for (int base = threadIdx.x; base < total; base += 8 * kLmmThreads) {
        uint32_t q[8];
        float sc[8], mn[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int item = min(base + u * kLmmThreads, total - 1);
            const int k = item / groups, cg4 = item - k * groups;
            const size_t I = static_cast<size_t>(k0 + k);
            const int c = c0 + cg4 * 4;
            q[u] = ld_stream_u32(t.codes + I * t.cols + c);
            if (MODE == 0) {
                sc[u] = __ldg(static_cast<const float*>(t.scale) + I * nb + c / t.gs);
                mn[u] = __ldg(t.mn + I * nb + c / t.gs);
            } else {
                sc[u] = __half2float(__ldg(static_cast<const __half*>(t.scale) + I));
                mn[u] = 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int item = base + u * kLmmThreads;
            if (item >= total) break;
            const int k = item / groups, cg4 = item - k * groups;
            float w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t byte = (q[u] >> (8 * e)) & 0xFFu;
                const float v = MODE == 0 ? __fadd_rn(__fmul_rn(static_cast<float>(byte), sc[u]), mn[u])
                                          : __fmul_rn(static_cast<float>(static_cast<int8_t>(byte)), sc[u]);
                w[e] = dense_param_rounding(v);
            }
            *reinterpret_cast<uint2*>(wk + k * pitch + cg4 * 4) = pack4h(w);
        }
    }
}
__device__ __forceinline__ void stage_wt_any(const QView& t, int k0, int kc, int c0, int nc, __half* wt, int pitch) {
    switch (lora_mode(t)) {
        case 0: stage_wt<0>(t, k0, kc, c0, nc, wt, pitch); break;
        case 1: stage_wt<1>(t, k0, kc, c0, nc, wt, pitch); break;
        default: stage_wt<2>(t, k0, kc, c0, nc, wt, pitch); break;
    }
}

// rows [0, nn) x columns [k0, k0 + kc) of src [*, ld] fp32 -> hi / lo [MT * 16][pitch] fp16 (rows beyond nn: zero)
__device__ __forceinline__ void stage_split(const float* src, long long ld, int nn, int rows_pad, int k0, int kc,
                                            __half* hi, __half* lo, int pitch) {
    const int g4 = kc >> 2, total = rows_pad * g4;
    for (int base = threadIdx.x; base < total; base += 8 * kLmmThreads) {      // 8 loads in flight per thread
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int item = base + u * kLmmThreads;
            const int n = item / g4, k4 = item - n * g4;
            v[u] = (item < total && n < nn) ? __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(n) * ld + k0) + k4)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int item = base + u * kLmmThreads;
            if (item >= total) break;
            const int n = item / g4, k4 = item - n * g4;
            uint2 h, l;
            split4(v[u], h, l);
            *reinterpret_cast<uint2*>(hi + n * pitch + 4 * k4) = h;
            *reinterpret_cast<uint2*>(lo + n * pitch + 4 * k4) = l;
        }
    }
}

// B fragments of a k16 step for two adjacent 8-column tiles from wk[k][n] (n contiguous): the four 8x8
// matrices (k 0-7 | 8-15) x (n 0-7 | 8-15), transposed on the way into the registers
__device__ __forceinline__ void ldsm_x4_trans(const __half* wk, int pitch, int kk, int n_base, int lane, uint32_t (&b)[2][2]) {
    const int m = lane >> 3, r = lane & 7;
    const __half* p = wk + (kk + (m & 1) * 8 + r) * pitch + n_base + (m >> 1) * 8;
    const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(b[0][0]), "=r"(b[0][1]), "=r"(b[1][0]), "=r"(b[1][1])
                 : "r"(addr));
}

// one k16 step: c[mi][ni] += A(m-tile mi) * B(n-tile ni), hi and lo halves of A; NI = 1 or 2 8-column
// tiles starting at column n_base of wk (both are loaded; one may go unused)
template <int MI, int NI>
__device__ __forceinline__ void lmm_step(float (&c)[MI][NI][4], const __half* ahi, const __half* alo, int apitch,
                                         const __half* wk, int wpitch, int n_base, int kk, int lane) {
    const int g = lane >> 2, t = lane & 3;
    uint32_t b[2][2];
    ldsm_x4_trans(wk, wpitch, kk, n_base, lane, b);
#pragma unroll
    for (int mi = 0; mi < MI; ++mi) {
        uint32_t ah[4], al[4];
        const int o0 = (mi * 16 + g) * apitch + kk + 2 * t, o1 = o0 + 8 * apitch;
        ah[0] = *reinterpret_cast<const uint32_t*>(ahi + o0); ah[1] = *reinterpret_cast<const uint32_t*>(ahi + o1);
        ah[2] = *reinterpret_cast<const uint32_t*>(ahi + o0 + 8); ah[3] = *reinterpret_cast<const uint32_t*>(ahi + o1 + 8);
        al[0] = *reinterpret_cast<const uint32_t*>(alo + o0); al[1] = *reinterpret_cast<const uint32_t*>(alo + o1);
        al[2] = *reinterpret_cast<const uint32_t*>(alo + o0 + 8); al[3] = *reinterpret_cast<const uint32_t*>(alo + o1 + 8);
#pragma unroll
        for (int ni = 0; ni < NI; ++ni) {
            lmm_mma(c[mi][ni], ah, b[ni][0], b[ni][1]);
            lmm_mma(c[mi][ni], al, b[ni][0], b[ni][1]);
        }
    }
}

// MT: 16-stream tiles per stream group (1, 2, 4)
template <int MT>
__global__ void __launch_bounds__(kLmmThreads) lora_down_mma_kernel(const LoraMmaArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = blockIdx.x;                                  // K slice = rank in the cluster
    const int br = static_cast<int>(blockIdx.y) % a.n_br, tg0 = static_cast<int>(blockIdx.y) / a.n_br;
    const int tg_step = static_cast<int>(gridDim.y) / a.n_br;
    const QView& t = a.t1[br];
    const int c0 = blockIdx.z * kLmmRC;
    const int kc = a.D / kLmmSlices, k0 = rank * kc;
    const int pitch = kc + kLmmPad;
    constexpr int WP = kLmmRC + kLmmPad;                          // pitch of a weight row (32 rank columns)
    __half* xhi = reinterpret_cast<__half*>(smem);
    __half* xlo = xhi + MT * 16 * pitch;
    __half* wt = xlo + MT * 16 * pitch;                           // [kc][WP]
    float* part = reinterpret_cast<float*>(wt + kc * WP);         // [MT * 16][kLmmRC + 1]
    constexpr int PP = kLmmRC + 1;
    const bool active = c0 < t.cols;                              // the whole cluster shares branch and column group
    pdl_launch_dependents();
    if (active && t.cols - c0 < kLmmRC)                           // ragged rank: the missing columns read as zero
        for (int i = threadIdx.x; i < kc * WP; i += kLmmThreads) wt[i] = __float2half_rn(0.f);
    __syncthreads();
    if (active) stage_wt_any(t, k0, kc, c0, min(kLmmRC, t.cols - c0), wt, WP);
    pdl_wait();
    for (int tg = tg0; tg < a.n_groups; tg += tg_step) {          // the staged weights serve every stream group of this CTA
    const int n0 = tg * MT * 16, nn = min(MT * 16, a.n_tokens - n0);
    if (active) stage_split(a.x[br] + static_cast<size_t>(n0) * a.ldx, a.ldx, nn, MT * 16, k0, kc, xhi, xlo, pitch);
    __syncthreads();
    if (active) {
        // 8 warps = MT m-tiles x (8 / MT) groups of the four 8-column tiles
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
        // 2 * MT (stream tile, 16-column half) pairs over the 8 warps; spare warps split nothing further
        constexpr int NI = 2;
        const int mi = warp % MT, ngi = warp / MT;
        if (ngi * NI < 4) {
            float c[1][NI][4];
#pragma unroll
            for (int ni = 0; ni < NI; ++ni) c[0][ni][0] = c[0][ni][1] = c[0][ni][2] = c[0][ni][3] = 0.f;
            for (int kk = 0; kk < kc; kk += 16)
                lmm_step<1, NI>(c, xhi + mi * 16 * pitch, xlo + mi * 16 * pitch, pitch, wt, WP, ngi * 16, kk, lane);
#pragma unroll
            for (int ni = 0; ni < NI; ++ni) {
                const int col = (ngi * NI + ni) * 8 + 2 * tq, row = mi * 16 + g;
                part[row * PP + col] = c[0][ni][0];
                part[row * PP + col + 1] = c[0][ni][1];
                part[(row + 8) * PP + col] = c[0][ni][2];
                part[(row + 8) * PP + col + 1] = c[0][ni][3];
            }
        }
    }
    cluster.sync();
    if (active) {
        const int total = nn * kLmmRC, per = (total + kLmmSlices - 1) / kLmmSlices;
        const int lo = rank * per, hi = min(total, lo + per);
        for (int idx = lo + threadIdx.x; idx < hi; idx += kLmmThreads) {
            const int n = idx / kLmmRC, col = idx - n * kLmmRC;
            if (c0 + col >= t.cols) continue;
            float pv[kLmmSlices];
#pragma unroll
            for (int k = 0; k < kLmmSlices; ++k) pv[k] = cluster.map_shared_rank(part, k)[n * PP + col];
            float v = 0.f;
#pragma unroll
            for (int k = 0; k < kLmmSlices; ++k) v += pv[k];
            if (a.act[br] == 1) v = tanhf(v);
            else if (a.act[br] == 2) v = sigmoidf_(v);
            a.h[(static_cast<size_t>(br) * a.n_stride + n0 + n) * a.max_rank + c0 + col] = v;
        }
    }
    cluster.sync();          // nobody overwrites or leaves while a peer still reads its partial sums
    }
}

template <int MT>
__global__ void __launch_bounds__(kLmmThreads) lora_up_mma_kernel(const LoraMmaArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int br = static_cast<int>(blockIdx.y) % a.n_br, tg0 = static_cast<int>(blockIdx.y) / a.n_br;
    const int tg_step = static_cast<int>(gridDim.y) / a.n_br;
    const QView& t = a.t2[br];
    const int r = t.rows, c0 = blockIdx.x * kLmmUpCols;
    const int pitch = r + kLmmPad;
    constexpr int WP = kLmmUpCols + kLmmPad;
    __half* hhi = reinterpret_cast<__half*>(smem);
    __half* hlo = hhi + MT * 16 * pitch;
    __half* wt = hlo + MT * 16 * pitch;                           // [r][WP]
    pdl_launch_dependents();
    stage_wt_any(t, 0, r, c0, kLmmUpCols, wt, WP);
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    for (int tg = tg0; tg < a.n_groups; tg += tg_step) {          // the staged weights serve every stream group of this CTA
    const int n0 = tg * MT * 16, nn = min(MT * 16, a.n_tokens - n0);
    __syncthreads();                                               // the previous group's operands have been read
    stage_split(a.h + (static_cast<size_t>(br) * a.n_stride + n0) * a.max_rank, a.max_rank, nn, MT * 16, 0, r, hhi, hlo, pitch);
    __syncthreads();
    // warp: 16 of the CTA's columns (warp % NPW) x a share of the stream tiles (warp / NPW)
    constexpr int NPW = kLmmUpCols / 16, MH = 8 / NPW, MI = MT >= MH ? MT / MH : 1;
    const int np = warp % NPW, mh = warp / NPW;
    if (mh * MI >= MT) continue;                                   // few streams: spare warps have no tile (they still meet the barriers above)
    float c[MI][2][4];
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) c[mi][ni][0] = c[mi][ni][1] = c[mi][ni][2] = c[mi][ni][3] = 0.f;
    for (int kk = 0; kk < r; kk += 16)
        lmm_step<MI, 2>(c, hhi + mh * MI * 16 * pitch, hlo + mh * MI * 16 * pitch, pitch, wt, WP, np * 16, kk, lane);
    float* y = a.y[br] + static_cast<size_t>(n0) * a.ldy + c0 + np * 16;
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {
            const int row = (mh * MI + mi) * 16 + g, col = ni * 8 + 2 * tq;
            if (row < nn) *reinterpret_cast<float2*>(y + static_cast<size_t>(row) * a.ldy + col) = make_float2(c[mi][ni][0], c[mi][ni][1]);
            if (row + 8 < nn) *reinterpret_cast<float2*>(y + static_cast<size_t>(row + 8) * a.ldy + col) = make_float2(c[mi][ni][2], c[mi][ni][3]);
        }
    }
}

namespace {

template <typename K>
int lmm_attr(K kernel, size_t smem) {
    if (smem <= 48 * 1024) return RWKVQ_OK;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kLmmMaxSmem);
    if (e != cudaSuccess) return fail(RWKVQ_E_LIMIT, "lora_mma: shared memory attribute: %s", cudaGetErrorString(e));
    return RWKVQ_OK;
}

template <int MT>
int launch_lmm(LoraMmaArgs& a, int groups, int max_cols, cudaStream_t s) {
    a.n_groups = groups;
    const int gy_down = std::min(groups, 4), gy_up = std::min(groups, 8);      // CTAs walk the remaining groups
    const int kc = a.D / kLmmSlices;
    const size_t smem_d = (static_cast<size_t>(2 * MT * 16) * (kc + kLmmPad) + static_cast<size_t>(kc) * (kLmmRC + kLmmPad)) * sizeof(__half) +
                          static_cast<size_t>(MT * 16) * (kLmmRC + 1) * sizeof(float);
    const size_t smem_u = (static_cast<size_t>(2 * MT * 16) * (a.max_rank + kLmmPad) +
                           static_cast<size_t>(a.max_rank) * (kLmmUpCols + kLmmPad)) * sizeof(__half);
    if (smem_d > static_cast<size_t>(kLmmMaxSmem) || smem_u > static_cast<size_t>(kLmmMaxSmem))
        return fail(RWKVQ_E_LIMIT, "lora_mma: %zu / %zu bytes of shared memory", smem_d, smem_u);
    int rc = lmm_attr(lora_down_mma_kernel<MT>, smem_d);
    if (rc) return rc;
    rc = lmm_attr(lora_up_mma_kernel<MT>, smem_u);
    if (rc) return rc;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(kLmmSlices, a.n_br * gy_down, (a.max_rank + kLmmRC - 1) / kLmmRC);
    cfg.blockDim = dim3(kLmmThreads);
    cfg.dynamicSmemBytes = smem_d;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kLmmSlices; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, lora_down_mma_kernel<MT>, a);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "lora_down_mma: %s", cudaGetErrorString(e));
    e = launch_pdl(lora_up_mma_kernel<MT>, dim3(max_cols / kLmmUpCols, a.n_br * gy_up), dim3(kLmmThreads), smem_u, s, a);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "lora_up_mma: %s", cudaGetErrorString(e));
    return RWKVQ_OK;
}

}  // namespace

// Whether the tensor-core pair serves these shapes: D a multiple of 128 (slices of D / 8 columns,
// whole k16 steps), every rank a multiple of 16 up to 512, and one output width for all branches, a
// multiple of the 32-column output tiles (D itself, or a rank's share of it in a head-sharded model).
bool lora_mma_ok(const rwkvq_qtensor* const* t1, const rwkvq_qtensor* const* t2, int n_br, int D) {
    if (D % 128 != 0) return false;
    for (int i = 0; i < n_br; ++i) {
        const int r = t1[i]->cols;
        if (t1[i]->rows != D || t2[i]->rows != r || r % 16 != 0 || r > 512 || r < 16) return false;
        if (t2[i]->cols != t2[0]->cols || t2[i]->cols % kLmmUpCols != 0 || t2[i]->cols < kLmmUpCols) return false;
    }
    return true;
}

// y_br = act_br(x_br @ W1_br) @ W2_br for n_br branches and B streams; h: scratch of
// 4 * n_stride * max_rank floats with n_stride >= B rounded up to the stream-group size.
int launch_lora_pair_mma(const rwkvq_qtensor* const* t1, const rwkvq_qtensor* const* t2, const float* const* xs,
                         float* const* ys, const int* acts, int n_br, int B, int D, int max_rank, float* h, int n_stride,
                         cudaStream_t s) {
    LoraMmaArgs a{};
    int max_cols = 0, mr = 0;
    for (int i = 0; i < n_br; ++i) {
        a.t1[i] = make_view(*t1[i]); a.t2[i] = make_view(*t2[i]);
        a.x[i] = xs[i]; a.y[i] = ys[i]; a.act[i] = acts[i];
        max_cols = t2[i]->cols > max_cols ? t2[i]->cols : max_cols;
        mr = t1[i]->cols > mr ? t1[i]->cols : mr;
    }
    a.h = h; a.ldx = D; a.ldy = max_cols; a.n_tokens = B; a.n_stride = n_stride; a.max_rank = max_rank; a.n_br = n_br; a.D = D;
    RWKVQ_REQUIRE(mr <= max_rank, RWKVQ_E_SHAPE, "lora_mma: rank %d above the model's max_rank %d", mr, max_rank);
    if (B <= 16) return launch_lmm<1>(a, 1, max_cols, s);
    if (B <= 32) return launch_lmm<2>(a, 1, max_cols, s);
    return launch_lmm<4>(a, (B + 63) / 64, max_cols, s);
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" size_t rwkvq_lora_pair_workspace_bytes(int N, int max_rank) {
    if (N < 1 || max_rank < 1) return 0;
    return static_cast<size_t>(4) * (((N + 63) / 64) * 64) * max_rank * sizeof(float);
}

extern "C" int rwkvq_lora_pair(const rwkvq_qtensor* t1_host, const rwkvq_qtensor* t2_host, int n_br,
                               const float* const* xs_host, float* const* ys_host, const int* acts_host, int N, int D,
                               void* workspace, size_t workspace_bytes, void* stream) {
    RWKVQ_REQUIRE(t1_host && t2_host && xs_host && ys_host && acts_host && workspace, RWKVQ_E_NULL, "rwkvq_lora_pair: null pointer");
    RWKVQ_REQUIRE(n_br >= 1 && n_br <= 4 && N >= 1, RWKVQ_E_SHAPE, "rwkvq_lora_pair: %d branches, %d rows", n_br, N);
    const rwkvq_qtensor* t1[4];
    const rwkvq_qtensor* t2[4];
    int max_rank = 0;
    for (int i = 0; i < n_br; ++i) {
        int rc = validate_qtensor(&t1_host[i], "rwkvq_lora_pair(down)");
        if (rc) return rc;
        rc = validate_qtensor(&t2_host[i], "rwkvq_lora_pair(up)");
        if (rc) return rc;
        RWKVQ_REQUIRE(xs_host[i] && ys_host[i], RWKVQ_E_NULL, "rwkvq_lora_pair: x or y of branch %d is null", i);
        RWKVQ_REQUIRE(aligned(xs_host[i], 16) && aligned(ys_host[i], 16), RWKVQ_E_ALIGN, "rwkvq_lora_pair: rows must be 16-byte aligned");
        RWKVQ_REQUIRE(acts_host[i] >= 0 && acts_host[i] <= 2, RWKVQ_E_DTYPE, "rwkvq_lora_pair: activation %d", acts_host[i]);
        t1[i] = &t1_host[i]; t2[i] = &t2_host[i];
        max_rank = t1_host[i].cols > max_rank ? t1_host[i].cols : max_rank;
    }
    RWKVQ_REQUIRE(lora_mma_ok(t1, t2, n_br, D), RWKVQ_E_SHAPE,
                  "rwkvq_lora_pair: needs D %% 128 == 0, every rank a multiple of 16 up to 512, W1 [D, r], W2 [r, C] with one C %% 32 == 0");
    RWKVQ_REQUIRE(aligned(workspace, 16) && workspace_bytes >= rwkvq_lora_pair_workspace_bytes(N, max_rank), RWKVQ_E_LIMIT,
                  "rwkvq_lora_pair: workspace of %zu bytes, %zu needed (16-byte aligned)", workspace_bytes,
                  rwkvq_lora_pair_workspace_bytes(N, max_rank));
    int rc = launch_lora_pair_mma(t1, t2, xs_host, ys_host, acts_host, n_br, N, D, max_rank, static_cast<float*>(workspace),
                                  ((N + 63) / 64) * 64, static_cast<cudaStream_t>(stream));
    return rc ? rc : check_launch("rwkvq_lora_pair");
}
