// Whole-token decode for one stream as ONE persistent cooperative kernel.
//
// The launch-chain decode step (rwkvq_decode_step) spends most of a token in launch
// and drain gaps: ~220 dependent kernels of a few microseconds each against ~130 us of
// HBM time.  Here the token is a short program of stages, interpreted by 2 CTAs per SM
// that stay resident; stages are separated by a grid-wide barrier (one atomic + a
// bounded spin on an L2 word) instead of a kernel boundary, and because the weights do
// not depend on the activations every warp issues the loads of its first weight
// fragment of the NEXT stage before it waits at the barrier, so the HBM stream keeps
// running across stage boundaries.
//
// Stages per layer (math: backends/metal/quant_model.py:638-728, 803-836):
//   S1  [LN1 + token shift + lerps, recomputed by every CTA] r/k/v GEMVs; the spare
//       CTAs compute the LoRA down projections as row-chunk partial sums
//   S2  one CTA per head: LoRA up projections of the head's 64 columns, decay/gates,
//       one WKV-7 step, group norm, bonus, gate
//   S3  output projection + residual
//   S4  [LN2 + token shift + lerp] ffn key GEMV, relu^2
//   S5  ffn value GEMV, K split over CTA pairs; the partial sums are added to the
//       residual stream by the next stage's prologue
// then [LN_out] head GEMV, and a two-stage argmax.  The embedding row and LN0 are part
// of the first stage's prologue.
//
// Every wait is bounded: a barrier that does not complete within kBarrierSpinLimit polls
// records RWKVQ_E_TIMEOUT in the status word and the CTA returns; the status is sticky
// (later launches return at once) until the decoder is initialised again.
#include <cooperative_groups.h>

#include <vector>

#include "rwkvq_decode_parts.cuh"
#include "rwkvq_gemv_mma.cuh"

namespace rwkvq {

constexpr int kPThreads = 256;
constexpr int kPMaxD = 4096;             // n_embd (registers of the LN prologue)
constexpr int kPMaxSlice = 8192;         // longest activation slice one CTA prepares
constexpr int kPMaxRank = 1024;          // sum of the LoRA ranks of a layer
constexpr int kPLoraRows = 64;           // rows of a LoRA down chunk
constexpr unsigned int kBarrierSpinLimit = 1u << 21;
constexpr int kUpSlotsMax = 12;

enum OpType { OP_GEMV = 0, OP_TMIX = 1, OP_ARGMAX_PART = 2, OP_ARGMAX_FINAL = 3 };
enum InKind { IN_VEC = 0, IN_LN = 1 };

// v[i] = f(resid[i] + sum_z part[z * stride + i]),  f = relu^2 or identity
struct VecSrc {
    const float* resid;
    const float* part;
    int n_parts, stride, relu2, pad_;
};

struct alignas(16) Op {
    int type;
    // ---- OP_GEMV: n_mats same-shape matrices; CTA unit = (matrix, group of wt tiles, K slice)
    int layout, n_mats, rows, cols, n_tiles, n_iters;
    int wt, wk, ks, n_groups, n_units, rows_padded, epilogue;
    int in_kind, has_emb;
    int mix_row[3];
    int n_lora, lora_chunks, lora_stride, lora_cg, lora_rows;
    int up_slots, slot_br[kUpSlotsMax], off64[4];
    int lora_mix_row[4], lora_off[4], lora_act[4];
    int D, H, layer0, V;
    QView t[3];
    QView l[4];                 // OP_GEMV: LoRA down matrices;  OP_TMIX: LoRA up matrices
    QView emb;
    VecSrc src;
    const float *ln_w, *ln_b, *mix, *ln0_w, *ln0_b;
    float *shift, *x_out;
    const long long* token;
    float* y[3];
    const float* resid_out;
    float* part_out;
    float* lora_part;           // [chunks][lora_stride]
    // ---- OP_TMIX
    const float *r, *k, *v, *w0, *a0, *v0, *k_k, *k_a, *r_k, *lnx_w, *lnx_b;
    float *v_first, *state, *og;
    // ---- OP_ARGMAX_*
    const float* logits;
    float* pv;
    int* pi;
    long long* next_token;
    long long* token_feed;
    int n_parts_argmax, pad2_;
};
static_assert(sizeof(Op) % 16 == 0, "Op is copied to shared memory as 16-byte words");

// sync[0] arrival counter (monotonic), sync[1] counter value at the start of a launch,
// sync[2] status (0 ok), sync[3] number of barriers passed (diagnostic)
// Polling load: relaxed (an acquire load would make the SM drop its L1 lines on every poll,
// which slows the CTA that shares the SM and is still working); the fence after the loop
// orders the reads that follow.
__device__ __forceinline__ unsigned int ld_poll_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Returns false when the wait ran out (status recorded); uniform over the CTA.
__device__ __forceinline__ bool grid_barrier(unsigned int* sync, unsigned int& epoch, int* s_flag) {
    __syncthreads();
    epoch += gridDim.x;
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(sync, 1u);
        unsigned int polls = 0;
        int ok = 1;
        while (static_cast<int>(ld_poll_u32(sync) - epoch) < 0) {
            if (++polls > kBarrierSpinLimit) { ok = 0; break; }
            __nanosleep(32);
        }
        if (!ok) atomicExch(reinterpret_cast<int*>(sync + 2), RWKVQ_E_TIMEOUT);
        __threadfence();
        *s_flag = ok;
    }
    __syncthreads();
    return *s_flag != 0;
}

__device__ __forceinline__ void copy_op(const Op* src, Op* dst) {
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(Op) / 16); i += kPThreads) d[i] = __ldg(s + i);
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Asynchronous global -> shared copies (no registers held while the data is in flight).
// 16-byte copies go through L2 only (.cg): safe for data written by other CTAs before the
// last grid barrier; 4-byte copies (.ca) are used for weights and parameters only.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem))), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem))), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Shared memory of a CTA, carved from one dynamic allocation.
struct PSmem {
    Op* op;            // [2]
    int8_t* dig;       // [3][slice]      (tmix: LoRA-up scratch)
    float* xs16;       // [slice / 16]
    float* xn;         // [D]  normalised row (LoRA chunks; CTA 0 keeps it for the deferred shift write)
    float* prev;       // [D]
    float* red;        // [2][128] + [32]
    int* flag;
    unsigned long long* trace;   // this CTA's 8 timeline slots of the current stage, or nullptr
};
__device__ __forceinline__ void mark(const PSmem& sm, int k) {
    if (sm.trace && threadIdx.x == 0) sm.trace[k] = global_ns();
}
// the same once `v` (the result of a load) has arrived
__device__ __forceinline__ void mark_after(const PSmem& sm, int k, float v) {
    if (sm.trace && threadIdx.x == 0) {
        float t;
        asm volatile("mov.f32 %0, %1;" : "=f"(t) : "f"(v));
        sm.trace[k] = global_ns() + (t == 1.2345e-30f ? 1 : 0);
    }
}

__device__ __forceinline__ float sum4(const float4& v) { return (v.x + v.y) + (v.z + v.w); }
__device__ __forceinline__ float4 add4(const float4& a, const float4& b) {
    return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}
__device__ __forceinline__ float4 relu2_4(float4 v) {
    v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
    v.x *= v.x; v.y *= v.y; v.z *= v.z; v.w *= v.w;
    return v;
}
__device__ __forceinline__ float4 zero4() { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ float4 lerp4(const float4& xn, const float4& pv, const float4& m) {
    return make_float4(xn.x + (pv.x - xn.x) * m.x, xn.y + (pv.y - xn.y) * m.y, xn.z + (pv.z - xn.z) * m.z,
                       xn.w + (pv.w - xn.w) * m.w);
}

// One dequantised element in the loader's precision; kept out of line (the generic decoder
// is large and only the embedding row and odd LoRA layouts need it).
__device__ __noinline__ float decode_rounded(const QView& t, int r, int c) { return dense_param_rounding(decode_element(t, r, c)); }

// Elements e..e+3 of a vector source; the loads of the residual and of the first two
// partial-sum slices are issued together (fixed order of additions: resid + p0 + p1 + ...).
__device__ __forceinline__ float4 src_load4(const VecSrc& s, int e) {
    const float4 r = s.resid ? __ldcg(reinterpret_cast<const float4*>(s.resid + e)) : zero4();
    const float4 p0 = s.n_parts > 0 ? __ldcg(reinterpret_cast<const float4*>(s.part + e)) : zero4();
    const float4 p1 = s.n_parts > 1 ? __ldcg(reinterpret_cast<const float4*>(s.part + s.stride + e)) : zero4();
    float4 v = r;
    if (s.n_parts > 0) v = add4(v, p0);
    if (s.n_parts > 1) v = add4(v, p1);
    for (int z = 2; z < s.n_parts; ++z)
        v = add4(v, __ldcg(reinterpret_cast<const float4*>(s.part + static_cast<size_t>(z) * s.stride + e)));
    return s.relu2 ? relu2_4(v) : v;
}

// Two-pass LayerNorm (eps 1e-5) of the row held as x[k] = elements 4*(tid + 256k)..+3.
template <int NR>
__device__ __forceinline__ void ln_apply(float4 (&x)[NR], const float4 (&lw)[NR], const float4 (&lb)[NR], int D, float* red) {
    const int n4 = D >> 2, tid = threadIdx.x;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NR; ++k) s += (tid + k * kPThreads < n4) ? sum4(x[k]) : 0.f;
    const float mean = block_sum(s, red) / D;
    float s2 = 0.f;
#pragma unroll
    for (int k = 0; k < NR; ++k)
        if (tid + k * kPThreads < n4) {
            const float a = x[k].x - mean, bb = x[k].y - mean, c = x[k].z - mean, d = x[k].w - mean;
            s2 += (a * a + bb * bb) + (c * c + d * d);
        }
    const float inv = 1.0f / sqrtf(block_sum(s2, red) / D + 1e-5f);
#pragma unroll
    for (int k = 0; k < NR; ++k)
        if (tid + k * kPThreads < n4) {
            x[k].x = (x[k].x - mean) * inv * lw[k].x + lb[k].x;
            x[k].y = (x[k].y - mean) * inv * lw[k].y + lb[k].y;
            x[k].z = (x[k].z - mean) * inv * lw[k].z + lb[k].z;
            x[k].w = (x[k].w - mean) * inv * lw[k].w + lb[k].w;
        }
}

// The LN prologue of a stage.  Assembles the residual-stream row (embedding + LN0 on the
// first stage), stores it when this CTA is the designated writer, normalises it, and
// returns in registers (elements 4*(tid + 256k)..+3): xn the normalised row, pv the
// previous token's normalised row, mx the lerp coefficients of `mix_row` (zeros if none).
// Every load is issued before the first value is used: one memory round trip.
template <int NR>
__device__ __forceinline__ void ln_core(const Op& op, const PSmem& sm, int mix_row, float4 (&xn)[NR], float4 (&pv)[NR],
                                        float4 (&mx)[NR]) {
    const int D = op.D, n4 = D >> 2, tid = threadIdx.x;
    float* red = sm.red + 256;
    float4 lw[NR], lb[NR], r[NR], p0[NR], p1[NR];
    const VecSrc& s = op.src;
    const float4* mixp = (op.mix && mix_row >= 0) ? reinterpret_cast<const float4*>(op.mix + static_cast<size_t>(mix_row) * D) : nullptr;
#pragma unroll
    for (int k = 0; k < NR; ++k) {
        const int i = tid + k * kPThreads;
        const bool ok = i < n4;
        r[k] = (ok && !op.has_emb && s.resid) ? __ldcg(reinterpret_cast<const float4*>(s.resid) + i) : zero4();
        p0[k] = (ok && !op.has_emb && s.n_parts > 0) ? __ldcg(reinterpret_cast<const float4*>(s.part) + i) : zero4();
        p1[k] = (ok && !op.has_emb && s.n_parts > 1) ? __ldcg(reinterpret_cast<const float4*>(s.part + s.stride) + i) : zero4();
        pv[k] = (ok && op.shift) ? __ldcg(reinterpret_cast<const float4*>(op.shift) + i) : zero4();
        if (NR <= 2) {        // small rows: the parameters ride along with the activations
            lw[k] = ok ? __ldg(reinterpret_cast<const float4*>(op.ln_w) + i) : zero4();
            lb[k] = ok ? __ldg(reinterpret_cast<const float4*>(op.ln_b) + i) : zero4();
            mx[k] = (ok && mixp) ? __ldg(mixp + i) : zero4();
        }
    }
    if (op.has_emb) {
        long long tok = __ldcg(op.token);
        tok = tok < 0 ? 0 : (tok >= op.emb.rows ? op.emb.rows - 1 : tok);
        float4 w0[NR], b0[NR];
#pragma unroll
        for (int k = 0; k < NR; ++k) {
            const int i = tid + k * kPThreads;
            xn[k] = zero4(); w0[k] = zero4(); b0[k] = zero4();
            if (i < n4) {
                const int row = static_cast<int>(tok);
                xn[k].x = decode_rounded(op.emb, row, 4 * i);
                xn[k].y = decode_rounded(op.emb, row, 4 * i + 1);
                xn[k].z = decode_rounded(op.emb, row, 4 * i + 2);
                xn[k].w = decode_rounded(op.emb, row, 4 * i + 3);
                w0[k] = __ldg(reinterpret_cast<const float4*>(op.ln0_w) + i);
                b0[k] = __ldg(reinterpret_cast<const float4*>(op.ln0_b) + i);
            }
        }
        ln_apply<NR>(xn, w0, b0, D, red);
    } else {
#pragma unroll
        for (int k = 0; k < NR; ++k) {
            xn[k] = r[k];
            if (s.n_parts > 0) xn[k] = add4(xn[k], p0[k]);
            if (s.n_parts > 1) xn[k] = add4(xn[k], p1[k]);
            for (int z = 2; z < s.n_parts; ++z) {
                const int i = tid + k * kPThreads;
                if (i < n4) xn[k] = add4(xn[k], __ldcg(reinterpret_cast<const float4*>(s.part + static_cast<size_t>(z) * s.stride) + i));
            }
        }
    }
    if (op.x_out && blockIdx.x == 0) {
#pragma unroll
        for (int k = 0; k < NR; ++k) {
            const int i = tid + k * kPThreads;
            if (i < n4) __stcg(reinterpret_cast<float4*>(op.x_out) + i, xn[k]);
        }
    }
    if (NR > 2) {             // wide rows: registers are short, the parameters follow in a second round
#pragma unroll
        for (int k = 0; k < NR; ++k) {
            const int i = tid + k * kPThreads;
            const bool ok = i < n4;
            lw[k] = ok ? __ldg(reinterpret_cast<const float4*>(op.ln_w) + i) : zero4();
            lb[k] = ok ? __ldg(reinterpret_cast<const float4*>(op.ln_b) + i) : zero4();
            mx[k] = (ok && mixp) ? __ldg(mixp + i) : zero4();
        }
    }
    ln_apply<NR>(xn, lw, lb, D, red);
}

// Digits of the activation slice that CTA unit (mat, z) multiplies with.  Returns the
// factor that undoes the fixed-point scaling (NaN when the input is not finite, which
// turns every output of the stage into NaN).
template <int NR>
__device__ __forceinline__ void ln_input(const Op& op, const PSmem& sm, int mat, float4 (&xr)[kXRegs]) {
    float4 xn[NR], pv[NR], mx[NR];
    ln_core<NR>(op, sm, op.mix ? op.mix_row[mat] : -1, xn, pv, mx);
    const int n4 = op.D >> 2;
    const bool keep = blockIdx.x == 0 && op.shift != nullptr;       // deferred token-shift write
#pragma unroll
    for (int k = 0; k < NR; ++k) {
        const int i = threadIdx.x + k * kPThreads;
        if (i < n4) {
            xr[k] = op.mix ? lerp4(xn[k], pv[k], mx[k]) : xn[k];
            if (keep) reinterpret_cast<float4*>(sm.xn)[i] = xn[k];
        }
    }
}

__device__ __noinline__ float prepare_input(const Op& op, const PSmem sm, int mat, int z, int n_slice, int bits) {
    const int tid = threadIdx.x;
    float4 xr[kXRegs];
#pragma unroll
    for (int k = 0; k < kXRegs; ++k) xr[k] = zero4();
    if (op.in_kind == IN_LN) {
        if (op.D <= 2 * 4 * kPThreads) ln_input<2>(op, sm, mat, xr);
        else ln_input<4>(op, sm, mat, xr);
        mark(sm, 3);
    } else {
        const int e0 = z * n_slice, n4 = n_slice >> 2;
#pragma unroll
        for (int k = 0; k < kXRegs; ++k) {
            const int i = tid + k * kPThreads;
            if (i < n4) xr[k] = src_load4(op.src, e0 + 4 * i);
        }
        mark_after(sm, 7, xr[0].x);
    }
    bool finite;
    const float unscale = digits_from_regs(xr, n_slice, bits, sm.dig, sm.xs16, sm.red + 256, finite);
    return finite ? unscale : NAN;
}

// ------------------------------------------------------------------ GEMV stage
// CTA unit u -> (matrix, tile group, K slice); warp -> (tile of the group, K lane).
struct UnitPos { int mat, grp, z; };
__device__ __forceinline__ UnitPos unit_pos(const Op& op, int u) {
    UnitPos p;
    p.z = u % op.ks;
    const int mg = u / op.ks;
    p.grp = mg % op.n_groups;
    p.mat = mg / op.n_groups;
    return p;
}

// Loads of item j of unit u for this warp (nothing when the warp has no such item).
template <int L>
__device__ __forceinline__ void fetch_item(FragData& f, const Op& op, int u, int j) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int tl = warp / op.wk, kw = warp - tl * op.wk;
    const int ipu = op.n_iters / op.ks;
    const UnitPos p = unit_pos(op, u);
    const int tile = p.grp * op.wt + tl, itl = kw + j * op.wk;
    if (u < op.n_units && tile < op.n_tiles && itl < ipu) {
        const QView& q = op.t[p.mat];
        load_frag<L>(f, q, min(tile * 16 + g, q.rows - 1), min(tile * 16 + g + 8, q.rows - 1), p.z * ipu + itl, t);
    }
}

__device__ __forceinline__ void prefetch_first(const Op& op, FragData& f) {
    if (op.type != OP_GEMV) return;
    const int u = blockIdx.x;
    switch (op.layout) {
        case ML_SB6_4: fetch_item<ML_SB6_4>(f, op, u, 0); break;
        case ML_SB6_5: fetch_item<ML_SB6_5>(f, op, u, 0); break;
        case ML_SB6_6: fetch_item<ML_SB6_6>(f, op, u, 0); break;
        case ML_SYM6: fetch_item<ML_SYM6>(f, op, u, 0); break;
        case ML_RTN8: fetch_item<ML_RTN8>(f, op, u, 0); break;
        default: fetch_item<ML_SYM8>(f, op, u, 0); break;
    }
}

// ---- LoRA down projections: part[chunk][off_br + j] = sum_{i in chunk} x_br[i] * W1_br[i][j]
// with x_br = lerp(xn, prev, mix_br).  The rank columns of all branches are laid back to
// back; a LoRA unit is (row chunk, group of 32 columns).  256 threads = 32 row groups x 8
// column threads (4 columns each, all inside one branch).  The packed weights and the lerp
// coefficients are requested before the LN prologue runs, so they arrive behind it.

struct LoraRaw { uint32_t q; float s, m; };

// raw codes + scale (+ min) of 4 consecutive weights of stored row i at column c
__device__ __forceinline__ LoraRaw lora_raw4(const QView& t, int mode, int i, int c) {
    LoraRaw r;
    const size_t I = static_cast<size_t>(i);
    r.q = ld_stream_u32(t.codes + I * t.cols + c);
    if (mode == 0) {
        const int nb = (t.cols + t.gs - 1) / t.gs, blk = c / t.gs;
        r.s = __ldg(static_cast<const float*>(t.scale) + I * nb + blk);
        r.m = __ldg(t.mn + I * nb + blk);
    } else {
        r.s = __half2float(__ldg(static_cast<const __half*>(t.scale) + I));
        r.m = 0.f;
    }
    return r;
}
__device__ __forceinline__ void lora_cvt4(const LoraRaw& r, int mode, float (&w)[4]) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t b = (r.q >> (8 * k)) & 0xFFu;
        const float q = mode == 0 ? static_cast<float>(b) : static_cast<float>(static_cast<int8_t>(b));
        w[k] = dense_param_rounding(__fadd_rn(__fmul_rn(q, r.s), r.m));
    }
}

// Staging: every thread copies the words it will consume (codes, scale, min, lerp
// coefficient of each of its rows) into its own shared-memory slots with cp.async, so no
// register is held while they are in flight and no barrier is needed to read them back.
template <int NR>
__device__ __forceinline__ void ln_to_smem(const Op& op, const PSmem& sm) {
    float4 xn[NR], pv[NR], mx[NR];
    ln_core<NR>(op, sm, -1, xn, pv, mx);
    const int n4 = op.D >> 2;
#pragma unroll
    for (int k = 0; k < NR; ++k) {
        const int i = threadIdx.x + k * kPThreads;
        if (i < n4) { reinterpret_cast<float4*>(sm.xn)[i] = xn[k]; reinterpret_cast<float4*>(sm.prev)[i] = pv[k]; }
    }
    __syncthreads();
}

__device__ __noinline__ void run_lora_down(const Op& op, const PSmem sm, int lu) {
    const int chunk = lu / op.lora_cg, cg = lu - chunk * op.lora_cg;
    const int tid = threadIdx.x, rg = tid >> 3, ct = tid & 7;
    const int col = cg * 32 + ct * 4;                     // column in the concatenated rank space
    int br = 0;
    for (int b = 1; b < op.n_lora; ++b) br += (col >= op.lora_off[b]) ? 1 : 0;
    const QView& t = op.l[br];
    const int jc = col - op.lora_off[br];                 // column inside the branch
    const bool live = jc < t.cols;
    const int mode = lora_mode(t);
    const float* mix = op.mix + static_cast<size_t>(op.lora_mix_row[br]) * op.D;
    const int row0 = chunk * op.lora_rows;
    const int n_r = op.lora_rows >> 5;                    // rows per thread
    uint32_t* stage = reinterpret_cast<uint32_t*>(sm.dig);    // [n_r][4][256] words, slot (r, w) of thread tid
    if (live && mode == 0) {
        const int nb = (t.cols + t.gs - 1) / t.gs, blk = jc / t.gs;
        for (int r = 0; r < n_r; ++r) {
            const int i = row0 + rg + 32 * r;
            if (i < t.rows) {
                const size_t I = static_cast<size_t>(i);
                cp_async4(stage + (r * 4 + 0) * kPThreads + tid, t.codes + I * t.cols + jc);
                cp_async4(stage + (r * 4 + 1) * kPThreads + tid, static_cast<const float*>(t.scale) + I * nb + blk);
                cp_async4(stage + (r * 4 + 2) * kPThreads + tid, t.mn + I * nb + blk);
                cp_async4(stage + (r * 4 + 3) * kPThreads + tid, mix + i);
            }
        }
    }
    if (op.D <= 2 * 4 * kPThreads) ln_to_smem<2>(op, sm);
    else ln_to_smem<4>(op, sm);
    cp_async_wait_all();
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
        for (int r = 0; r < n_r; ++r) {
            const int i = row0 + rg + 32 * r;
            if (i >= t.rows) break;
            float w[4], mv;
            if (mode == 0) {
                LoraRaw raw;
                raw.q = stage[(r * 4 + 0) * kPThreads + tid];
                raw.s = __uint_as_float(stage[(r * 4 + 1) * kPThreads + tid]);
                raw.m = __uint_as_float(stage[(r * 4 + 2) * kPThreads + tid]);
                mv = __uint_as_float(stage[(r * 4 + 3) * kPThreads + tid]);
                lora_cvt4(raw, 0, w);
            } else if (mode == 1) {
                lora_cvt4(lora_raw4(t, 1, i, jc), 1, w);
                mv = __ldg(mix + i);
            } else {
                for (int k = 0; k < 4; ++k) w[k] = decode_rounded(t, i, jc + k);
                mv = __ldg(mix + i);
            }
            const float xn = sm.xn[i];
            const float xv = xn + (sm.prev[i] - xn) * mv;
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[k] = fmaf(xv, w[k], acc[k]);
        }
    }
    // 32 row groups -> one value per column, added in row-group order
    __syncthreads();
    float* red = reinterpret_cast<float*>(sm.dig);            // [32][32]
#pragma unroll
    for (int k = 0; k < 4; ++k) red[rg * 32 + ct * 4 + k] = acc[k];
    __syncthreads();
    if (tid < 32) {
        float v = 0.f;
#pragma unroll
        for (int g = 0; g < 32; ++g) v += red[g * 32 + tid];
        const int c = cg * 32 + tid;
        if (c < op.lora_stride) __stcg(op.lora_part + static_cast<size_t>(chunk) * op.lora_stride + c, v);
    }
}

// One GEMV stage for the CTA units of this CTA.  `nxt` holds the first fragment (loaded
// before the preceding barrier).  Returns true when this CTA kept a normalised row whose
// token-shift write is still due.
template <int L>
__device__ __forceinline__ bool run_gemv(const Op& op, const PSmem& sm, FragData& nxt) {
    using G = Geo<L>;
    const int c = blockIdx.x, NG = gridDim.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int wk = op.wk, wt = op.wt, ks = op.ks;
    const int tl = warp / wk, kw = warp - tl * wk;
    const int ipu = op.n_iters / ks;                          // iterations of one K slice
    const int ipt = kw < ipu ? (ipu - kw + wk - 1) / wk : 0;  // this warp's items per unit
    const int n_slice = ipu * G::KI;
    const bool keep_shift = c == 0 && op.in_kind == IN_LN && op.shift != nullptr;
    int fu = c, fj = 0;                                       // item held in nxt
    auto advance = [&]() { if (++fj >= ipt) { fj = 0; fu += NG; } };
    if (ipt > 0) advance();
    int prepared = -1, buf = 0;
    float unscale = 0.f;
    for (int u = c; u < op.n_units; u += NG, buf ^= 1) {
        const UnitPos p = unit_pos(op, u);
        if (p.mat * ks + p.z != prepared) {
            unscale = prepare_input(op, sm, p.mat, p.z, n_slice, x_bits<L>());
            prepared = p.mat * ks + p.z;
            mark(sm, 4);
        }
        const int tile = p.grp * wt + tl;
        float acc0 = 0.f, acc1 = 0.f;
        for (int j = 0; j < ipt; ++j) {
            const FragData cur = nxt;
            if (fu < op.n_units) fetch_item<L>(nxt, op, fu, fj);
            advance();
            if (tile < op.n_tiles) consume_frag<L>(cur, kw + j * wk, g, t, sm.dig, n_slice, sm.xs16, acc0, acc1);
        }
        mark(sm, 5);
        acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 1); acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 2);
        acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 1); acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 2);
        float* rb = sm.red + buf * 128;
        if (t == 0) { rb[warp * 16 + g] = acc0; rb[warp * 16 + g + 8] = acc1; }
        __syncthreads();
        if (threadIdx.x < wt * 16) {
            const int wtl = threadIdx.x >> 4, r = threadIdx.x & 15;
            const int row = (p.grp * wt + wtl) * 16 + r;
            float v = 0.f;
            for (int k = 0; k < wk; ++k) v += rb[(wtl * wk + k) * 16 + r];
            v = v * unscale;
            if (ks > 1) {
                if (row < op.rows_padded)
                    __stcg(op.part_out + (static_cast<size_t>(p.z) * op.n_mats + p.mat) * op.rows_padded + row, v);
            } else if (row < op.rows) {
                if (op.epilogue == RWKVQ_EPI_RELU2) { v = fmaxf(v, 0.f); v = v * v; }
                else if (op.epilogue == RWKVQ_EPI_ADD) v = __fadd_rn(v, __ldcg(op.resid_out + row));
                __stcg(op.y[p.mat] + row, v);
            }
        }
    }
    mark(sm, 6);
    return keep_shift;
}

// ------------------------------------------------------------------ time-mix stage
// One CTA per head.  Every independent load of the stage is requested up front (state,
// LoRA-down partial sums, the head's 64 columns of the four LoRA-up matrices, r/k/v):
// one memory round trip, then arithmetic.
//
// LoRA up: the rank rows of the branches are laid back to back with every branch padded
// to a multiple of 64 rows ("slots" of 64 rows, each inside one branch).  256 threads =
// 64 row threads x 4 column threads (16 columns each); a thread holds one row per slot.
constexpr int kUpSlots = kUpSlotsMax;

// Fixed part of the stage's shared memory; the staging areas follow it:
//   state [64][64] f32 | codes [slots * 64 rows][64 B] | scale, min [slots * 64] f32 |
//   partial sums [chunks][stride] f32
struct TmixSmem {
    float hs[kPMaxRank];          // activated LoRA hidden vectors, branches back to back (unpadded)
    float up[8][4][64];           // per warp and branch: sums over the warp's 8 row threads
    float yl[4][64];              // LoRA outputs of this head: w, a, g, v
    float sA[64], sW[64], sK[64], sB[64], sR[64], sV[64], sY[64];
};
__host__ __device__ inline size_t tmix_smem_bytes(int slots, int chunks, int stride) {
    return sizeof(TmixSmem) + 64 * 64 * 4 + static_cast<size_t>(slots) * 64 * (64 + 8) +
           static_cast<size_t>(chunks) * stride * 4;
}

__device__ __noinline__ void run_tmix(const Op& op, const PSmem sm) {
    const int hi = blockIdx.x, tid = threadIdx.x;
    if (hi >= op.H) return;
    TmixSmem& ts = *reinterpret_cast<TmixSmem*>(sm.dig);
    float* st_sm = reinterpret_cast<float*>(sm.dig + sizeof(TmixSmem));
    const int n_rows = op.up_slots * 64;
    uint8_t* code_sm = reinterpret_cast<uint8_t*>(st_sm + 64 * 64);
    float* s_sm = reinterpret_cast<float*>(code_sm + static_cast<size_t>(n_rows) * 64);
    float* m_sm = s_sm + n_rows;
    float* part_sm = m_sm + n_rows;
    float* red = sm.red + 256;
    // ---- requests: everything the stage reads, in flight at once
    float* state = op.state + static_cast<size_t>(hi) * 64 * 64;
#pragma unroll
    for (int i = 0; i < 4; ++i) cp_async16(st_sm + (tid + i * kPThreads) * 4, state + (tid + i * kPThreads) * 4);
    for (int idx = tid; idx < n_rows * 4; idx += kPThreads) {
        const int row = idx >> 2, q = idx & 3, br = op.slot_br[row >> 6];
        const QView& t = op.l[br];
        const int r = row - op.off64[br];
        if (r < t.rows) cp_async16(code_sm + idx * 16, t.codes + static_cast<size_t>(r) * t.cols + hi * 64 + q * 16);
    }
    for (int row = tid; row < n_rows; row += kPThreads) {
        const int br = op.slot_br[row >> 6];
        const QView& t = op.l[br];
        const int r = row - op.off64[br];
        if (r < t.rows) {
            if (t.kind == RWKVQ_KIND_ASYM) {
                const int nb = (t.cols + t.gs - 1) / t.gs, blk = (hi * 64) / t.gs;
                cp_async4(s_sm + row, static_cast<const float*>(t.scale) + static_cast<size_t>(r) * nb + blk);
                cp_async4(m_sm + row, t.mn + static_cast<size_t>(r) * nb + blk);
            } else {
                s_sm[row] = __half2float(__ldg(static_cast<const __half*>(t.scale) + r));
                m_sm[row] = 0.f;
            }
        }
    }
    {
        const int n16 = (op.lora_chunks * op.lora_stride) >> 2;
        for (int idx = tid; idx < n16; idx += kPThreads) cp_async16(part_sm + idx * 4, op.lora_part + idx * 4);
    }
    float r_ = 0.f, k_ = 0.f, v_ = 0.f, vf_ = 0.f;
    if (tid < 64) {
        const int c = hi * 64 + tid;
        r_ = __ldcg(op.r + c); k_ = __ldcg(op.k + c); v_ = __ldcg(op.v + c);
        if (!op.layer0) vf_ = __ldcg(op.v_first + c);
    }
    cp_async_wait_all();
    __syncthreads();
    mark(sm, 3);
    // ---- LoRA hidden vectors: chunk partial sums added in chunk order, then the activation
    for (int j = tid; j < op.lora_stride; j += kPThreads) {
        float v = 0.f;
        for (int u = 0; u < op.lora_chunks; ++u) v += part_sm[u * op.lora_stride + j];
        int br = 0;
        for (int b = 1; b < op.n_lora; ++b) br += (j >= op.lora_off[b]) ? 1 : 0;
        if (op.lora_act[br] == 1) v = tanhf(v);
        else if (op.lora_act[br] == 2) v = sigmoidf_(v);
        ts.hs[j] = v;
    }
    __syncthreads();
    mark(sm, 4);
    // ---- LoRA up: 256 threads = 64 row threads x 4 column threads (16 columns each); per
    // branch, its slots of 64 rows, then a reduction over the row threads
    const int warp = tid >> 5, lane = tid & 31, jg = tid >> 2, cq = tid & 3;
    for (int br = 0; br < op.n_lora; ++br) {
        float acc[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) acc[k] = 0.f;
        const QView& t = op.l[br];
        const bool is_asym = t.kind == RWKVQ_KIND_ASYM;
        const float* hs = ts.hs + op.lora_off[br];
        for (int s = 0; s < op.up_slots; ++s) {
            if (op.slot_br[s] != br) continue;
            const int row = 64 * s + jg, r = row - op.off64[br];
            if (r < t.rows) {
                const float hv = hs[r], sc = s_sm[row], mn = m_sm[row];
                const uint4 q4 = *reinterpret_cast<const uint4*>(code_sm + static_cast<size_t>(row) * 64 + cq * 16);
                const uint32_t qw[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const uint32_t b = (qw[k >> 2] >> (8 * (k & 3))) & 0xFFu;
                    const float q = is_asym ? static_cast<float>(b) : static_cast<float>(static_cast<int8_t>(b));
                    acc[k] = fmaf(hv, dense_param_rounding(__fadd_rn(__fmul_rn(q, sc), mn)), acc[k]);
                }
            }
        }
        // lanes of a warp: 8 row threads x 4 column threads
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            acc[k] += __shfl_xor_sync(0xFFFFFFFFu, acc[k], 4);
            acc[k] += __shfl_xor_sync(0xFFFFFFFFu, acc[k], 8);
            acc[k] += __shfl_xor_sync(0xFFFFFFFFu, acc[k], 16);
        }
        if (lane < 4) {
#pragma unroll
            for (int k = 0; k < 16; ++k) ts.up[warp][br][lane * 16 + k] = acc[k];
        }
    }
    __syncthreads();
    {
        const int br = tid >> 6, cc = tid & 63;
        float v = 0.f;
        if (br < op.n_lora) {
#pragma unroll
            for (int w = 0; w < 8; ++w) v += ts.up[w][br][cc];
        }
        ts.yl[br][cc] = v;
    }
    __syncthreads();
    mark(sm, 5);
    // ---- decay, gates, kk, k and v updates (branch order: 0 w, 1 a, 2 g, 3 v)
    float kk = 0.f, av = 0.f;
    if (tid < 64) {
        const int c = hi * 64 + tid;
        float v = v_;
        const float w = expf(-0.606531f * sigmoidf_(ts.yl[0][tid] + op.w0[c]));
        av = sigmoidf_(ts.yl[1][tid] + op.a0[c]);
        kk = k_ * op.k_k[c];
        const float k2 = k_ * (1.0f + (av - 1.0f) * op.k_a[c]);
        if (op.layer0) __stcg(op.v_first + c, v);
        else v = v + (vf_ - v) * sigmoidf_(ts.yl[3][tid] + op.v0[c]);
        ts.sW[tid] = w; ts.sK[tid] = k2; ts.sR[tid] = r_; ts.sV[tid] = v;
    }
    const float n2 = block_sum(tid < 64 ? kk * kk : 0.f, red);
    if (tid < 64) {
        const float kn = kk / sqrtf(n2 + 1e-12f);
        ts.sA[tid] = -kn;
        ts.sB[tid] = kn * av;
    }
    __syncthreads();
    // ---- one WKV-7 step on the thread's 16 state columns
    const int dv = tid >> 2, part = tid & 3;
    float h[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 v4 = *reinterpret_cast<const float4*>(st_sm + dv * 64 + part * 16 + 4 * i);
        h[4 * i] = v4.x; h[4 * i + 1] = v4.y; h[4 * i + 2] = v4.z; h[4 * i + 3] = v4.w;
    }
    float sa = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) sa = fmaf(h[i], ts.sA[part * 16 + i], sa);
    sa += __shfl_xor_sync(0xFFFFFFFFu, sa, 1);
    sa += __shfl_xor_sync(0xFFFFFFFFu, sa, 2);
    const float vv = ts.sV[dv];
    float y = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int dk = part * 16 + i;
        h[i] = fmaf(ts.sW[dk], h[i], fmaf(vv, ts.sK[dk], sa * ts.sB[dk]));
        y = fmaf(h[i], ts.sR[dk], y);
    }
    y += __shfl_xor_sync(0xFFFFFFFFu, y, 1);
    y += __shfl_xor_sync(0xFFFFFFFFu, y, 2);
    float* hp = state + dv * 64 + part * 16;
#pragma unroll
    for (int i = 0; i < 4; ++i)
        *reinterpret_cast<float4*>(hp + 4 * i) = make_float4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
    if (part == 0) ts.sY[dv] = y;
    __syncthreads();
    mark(sm, 6);
    // ---- group norm over the head (two-pass), bonus, gate
    const float yv_ = tid < 64 ? ts.sY[tid] : 0.f;
    const float mean = block_sum(yv_, red) / 64.f;
    const float dc = tid < 64 ? yv_ - mean : 0.f;
    const float var = block_sum(dc * dc, red) / 64.f;
    const float dp = block_sum(tid < 64 ? ts.sR[tid] * ts.sK[tid] * op.r_k[hi * 64 + tid] : 0.f, red);
    if (tid < 64) {
        const int c = hi * 64 + tid;
        const float nrm = dc * (1.0f / sqrtf(var + 64e-5f));
        __stcg(op.og + c, (nrm * op.lnx_w[c] + op.lnx_b[c] + dp * ts.sV[tid]) * ts.yl[2][tid]);
    }
}

// ------------------------------------------------------------------ argmax stages
__device__ __noinline__ void run_argmax_part(const Op& op, const PSmem sm) {
    float* bv = sm.red;
    int* bi = reinterpret_cast<int*>(sm.red + 16);
    const int V = op.V, per = (V + gridDim.x - 1) / gridDim.x;
    const int lo = blockIdx.x * per, hi = min(lo + per, V);
    float best = -INFINITY;
    int idx = V;
    for (int i = lo + threadIdx.x; i < hi; i += kPThreads) argmax_combine(best, idx, __ldcg(op.logits + i), i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        argmax_combine(best, idx, __shfl_xor_sync(0xFFFFFFFFu, best, o), __shfl_xor_sync(0xFFFFFFFFu, idx, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kPThreads / 32; ++w) argmax_combine(best, idx, bv[w], bi[w]);
        __stcg(op.pv + blockIdx.x, best);
        __stcg(op.pi + blockIdx.x, idx);
    }
}

__device__ __noinline__ void run_argmax_final(const Op& op, const PSmem sm) {
    if (blockIdx.x != 0) return;
    float* bv = sm.red;
    int* bi = reinterpret_cast<int*>(sm.red + 16);
    float best = -INFINITY;
    int idx = op.V;
    for (int i = threadIdx.x; i < static_cast<int>(gridDim.x); i += kPThreads)
        argmax_combine(best, idx, __ldcg(op.pv + i), __ldcg(op.pi + i));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        argmax_combine(best, idx, __shfl_xor_sync(0xFFFFFFFFu, best, o), __shfl_xor_sync(0xFFFFFFFFu, idx, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kPThreads / 32; ++w) argmax_combine(best, idx, bv[w], bi[w]);
        const long long tok = idx < op.V ? idx : 0;
        if (op.next_token) *op.next_token = tok;
        if (op.token_feed) *op.token_feed = tok;
    }
}

// ------------------------------------------------------------------ the interpreter
struct PersistArgs {
    const Op* ops;
    int n_ops;
    unsigned int* sync;
    int work_bytes;        // digit / scratch region
    int D;
    // optional timeline: trace[(op * gridDim.x + cta) * 8 + {0 start, 1 work done, 2 barrier passed,
    // 3 row normalised, 4 input digits ready, 5 items consumed, 6 outputs written}]
    // in nanoseconds of the global timer; nullptr in normal operation
    unsigned long long* trace;
};

__device__ __forceinline__ void trace_mark(const PersistArgs& a, int op, int k) {
    if (a.trace && threadIdx.x == 0) a.trace[(static_cast<size_t>(op) * gridDim.x + blockIdx.x) * 8 + k] = global_ns();
}

__global__ void __launch_bounds__(kPThreads, 2) decode_persist_kernel(const PersistArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    PSmem sm;
    unsigned char* p = smem_raw;
    sm.op = reinterpret_cast<Op*>(p);                     p += 2 * sizeof(Op);
    sm.dig = reinterpret_cast<int8_t*>(p);                p += a.work_bytes;
    sm.xn = reinterpret_cast<float*>(p);                  p += a.D * sizeof(float);
    sm.prev = reinterpret_cast<float*>(p);                p += a.D * sizeof(float);
    sm.red = reinterpret_cast<float*>(p);                 p += (256 + 32) * sizeof(float);
    sm.flag = reinterpret_cast<int*>(p);
    sm.xs16 = nullptr;                                    // set per op (depends on the slice length)

    if (__ldcg(reinterpret_cast<const int*>(a.sync + 2)) != 0) return;      // sticky error of an earlier launch
    const long long clk0 = clock64();
    const unsigned long long ns0 = global_ns();
    unsigned int epoch = __ldcg(a.sync + 1);
    copy_op(a.ops, sm.op);
    __syncthreads();
    FragData nxt;
    prefetch_first(sm.op[0], nxt);
    float* pending_shift = nullptr;
    for (int i = 0; i < a.n_ops; ++i) {
        const Op& op = sm.op[i & 1];
        if (i + 1 < a.n_ops) copy_op(a.ops + i + 1, sm.op + ((i + 1) & 1));
        bool keep = false;
        sm.trace = a.trace ? a.trace + (static_cast<size_t>(i) * gridDim.x + blockIdx.x) * 8 : nullptr;
        trace_mark(a, i, 0);
        if (op.type == OP_GEMV) {
            const int c = blockIdx.x;
            if (c < op.n_units) {
                const int slice = op.cols / op.ks;
                sm.xs16 = reinterpret_cast<float*>(sm.dig + 3 * slice);
                switch (op.layout) {
                    case ML_SB6_4: keep = run_gemv<ML_SB6_4>(op, sm, nxt); break;
                    case ML_SB6_5: keep = run_gemv<ML_SB6_5>(op, sm, nxt); break;
                    case ML_SB6_6: keep = run_gemv<ML_SB6_6>(op, sm, nxt); break;
                    case ML_SYM6: keep = run_gemv<ML_SYM6>(op, sm, nxt); break;
                    case ML_RTN8: keep = run_gemv<ML_RTN8>(op, sm, nxt); break;
                    default: keep = run_gemv<ML_SYM8>(op, sm, nxt); break;
                }
            } else if (op.n_lora > 0 && c - op.n_units < op.lora_chunks * op.lora_cg) {
                run_lora_down(op, sm, c - op.n_units);
            }
        } else if (op.type == OP_TMIX) {
            run_tmix(op, sm);
        } else if (op.type == OP_ARGMAX_PART) {
            run_argmax_part(op, sm);
        } else {
            run_argmax_final(op, sm);
        }
        if (keep) pending_shift = op.shift;
        __syncthreads();                                  // the next op's descriptor is complete
        trace_mark(a, i, 1);
        if (i + 1 == a.n_ops) break;                      // nothing follows the last stage
        prefetch_first(sm.op[(i + 1) & 1], nxt);
        if (!grid_barrier(a.sync, epoch, sm.flag)) return;
        trace_mark(a, i, 2);
        if (pending_shift) {                              // every CTA has read the old row by now
            for (int k = threadIdx.x; k < (a.D >> 2); k += kPThreads)
                __stcg(reinterpret_cast<float4*>(pending_shift) + k, reinterpret_cast<const float4*>(sm.xn)[k]);
            pending_shift = nullptr;
            __syncthreads();
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        if (a.trace) {        // SM cycles and nanoseconds of the whole launch (slots 3, 4 of the last stage)
            unsigned long long* row = a.trace + (static_cast<size_t>(a.n_ops - 1) * gridDim.x) * 8;
            row[3] = static_cast<unsigned long long>(clock64() - clk0);
            row[4] = global_ns() - ns0;
        }
        a.sync[1] = epoch;                                // start value of the next launch
        a.sync[3] = static_cast<unsigned int>(a.n_ops);
    }
}

}  // namespace rwkvq

// ------------------------------------------------------------------ host side
using namespace rwkvq;

struct rwkvq_decoder {
    int n_ops, grid, smem, work_bytes, D, V;
    unsigned long long* trace;
    const Op* ops_dev;
    unsigned int* sync;
    long long* token;      // device slot: input token, overwritten with the greedy next token
    float* logits;
};

namespace {

int ki_of(int layout) { return layout <= ML_SB6_6 ? 256 : 128; }

// host mirror of lora_mode(): 0 asym / 1 per-row int8 with 4-column loads, 2 anything else
int lora_mode_host(const rwkvq_qtensor& t) {
    if (t.kind == RWKVQ_KIND_ASYM && (t.cols & 3) == 0) return 0;
    if (t.kind == RWKVQ_KIND_RTN && t.bits > 4 && (t.cols & 3) == 0) return 1;
    return 2;
}

// Work split of one GEMV stage over `grid` resident CTAs: the fewest waves of CTA units,
// then the shortest per-warp item chain; K is split across CTAs only when that helps.
void plan_split(Op& op, int grid, bool allow_ks) {
    const int tiles = op.n_tiles, iters = op.n_iters;
    double best = 1e30;
    for (int ks = 1; ks <= (allow_ks ? 4 : 1); ks <<= 1) {
        if (iters % ks) continue;
        if (op.cols / ks > kPMaxSlice) continue;
        for (int wt = 1; wt <= 8; wt <<= 1) {
            const int wk = 8 / wt, ipu = iters / ks;
            const int groups = (tiles + wt - 1) / wt;
            const int units = op.n_mats * groups * ks;
            const int waves = (units + grid - 1) / grid;
            const double cost = waves * ((ipu + wk - 1) / wk + 1.5) + 0.25 * (ks - 1);
            if (cost < best - 1e-9) {
                best = cost;
                op.wt = wt; op.wk = wk; op.ks = ks; op.n_groups = groups; op.n_units = units;
            }
        }
    }
}

struct Carver {
    char* base;
    size_t off = 0;
    template <typename T>
    T* take(size_t n) {
        T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
        off += ((n * sizeof(T) + 255) / 256) * 256;
        return p;
    }
};

struct Built {
    std::vector<Op> ops;
    size_t bytes = 0;
    int work_bytes = 0;
    Op* ops_dev = nullptr;
    unsigned int* sync = nullptr;
    long long* token = nullptr;
    float* logits = nullptr;
};

int gemv_op(Op& op, const rwkvq_qtensor* const* ts, int n_mats, int grid, bool allow_ks, const char* what) {
    op.type = OP_GEMV;
    op.n_mats = n_mats;
    op.layout = mma_layout_of(*ts[0]);
    for (int k = 0; k < n_mats; ++k) {
        int rc = validate_qtensor(ts[k], what);
        if (rc) return rc;
        RWKVQ_REQUIRE(mma_layout_of(*ts[k]) == op.layout && op.layout >= 0, RWKVQ_E_DTYPE,
                      "rwkvq_decoder: %s has no tensor-core GEMV layout (kind %d, %d bits, relayout %s)", what,
                      ts[k]->kind, ts[k]->bits, ts[k]->dev_meta || ts[k]->dev_planes ? "present" : "missing");
        RWKVQ_REQUIRE(ts[k]->rows == ts[0]->rows && ts[k]->cols == ts[0]->cols, RWKVQ_E_SHAPE,
                      "rwkvq_decoder: %s: fused matrices differ in shape", what);
        op.t[k] = make_view(*ts[k]);
    }
    op.rows = ts[0]->rows; op.cols = ts[0]->cols;
    op.n_tiles = (op.rows + 15) / 16;
    op.n_iters = op.cols / ki_of(op.layout);
    op.rows_padded = op.n_tiles * 16;
    plan_split(op, grid, allow_ks);
    RWKVQ_REQUIRE(op.n_units > 0, RWKVQ_E_LIMIT, "rwkvq_decoder: %s: no work split fits (cols %d)", what, op.cols);
    return RWKVQ_OK;
}

// Builds the stage program; with base == nullptr only sizes are computed.
int build_program(const rwkvq_model& m, float* const* wkv, float* const* tshift, float* const* cshift, int grid,
                  void* base, float* user_logits, Built& out) {
    const int D = m.n_embd, F = m.ffn_dim, V = m.vocab_size, H = D / 64;
    RWKVQ_REQUIRE(m.head_size == 64, RWKVQ_E_SHAPE, "rwkvq_decoder: head size %d, only 64 is built", m.head_size);
    RWKVQ_REQUIRE(D % 256 == 0 && D <= kPMaxD, RWKVQ_E_LIMIT, "rwkvq_decoder: n_embd %d (multiple of 256, at most %d)", D, kPMaxD);
    RWKVQ_REQUIRE(H <= grid, RWKVQ_E_LIMIT, "rwkvq_decoder: %d heads but only %d resident CTAs", H, grid);
    Carver cv{static_cast<char*>(base)};
    const int n_ops = m.n_layer * 5 + 3;
    out.ops_dev = cv.take<Op>(n_ops);
    out.sync = cv.take<unsigned int>(64);
    out.token = cv.take<long long>(1);
    float* xa = cv.take<float>(D);
    float* xb = cv.take<float>(D);
    float* rkv = cv.take<float>(3 * D);
    float* og = cv.take<float>(D);
    float* hffn = cv.take<float>(F);
    float* v_first = cv.take<float>(D);
    float* part = cv.take<float>(4 * static_cast<size_t>(((F > D ? F : D) + 15) / 16 * 16));
    float* lora_part = cv.take<float>(static_cast<size_t>(8) * kPMaxRank);     // at most 8 row chunks
    float* own_logits = cv.take<float>(V);
    float* logits = user_logits ? user_logits : own_logits;
    float* pv = cv.take<float>(grid);
    int* pi = cv.take<int>(grid);
    out.logits = logits;
    out.bytes = cv.off;

    int work = 0;
    auto need_work = [&](const Op& op) {
        const int slice = op.cols / op.ks;
        const int b = 3 * slice + 4 * (slice / 16);
        if (b > work) work = b;
    };
    out.ops.clear();
    VecSrc cur{};                        // where the residual stream row is at this point
    bool first = true;
    int rc = validate_qtensor(&m.emb, "rwkvq_decoder(emb)");
    if (rc) return rc;
    for (int l = 0; l < m.n_layer; ++l) {
        const rwkvq_layer& L = m.layers[l];
        const bool layer0 = l == 0;
        // ---- S1: r/k/v + LoRA down
        Op s1{};
        const rwkvq_qtensor* rkv_t[3] = {&L.Wr, &L.Wk, &L.Wv};
        rc = gemv_op(s1, rkv_t, 3, grid, false, "r/k/v");
        if (rc) return rc;
        RWKVQ_REQUIRE(s1.rows == D && s1.cols == D, RWKVQ_E_SHAPE, "rwkvq_decoder: r/k/v must be [%d, %d]", D, D);
        s1.in_kind = IN_LN; s1.D = D;
        s1.ln_w = L.ln1_w; s1.ln_b = L.ln1_b; s1.mix = L.x_mix; s1.shift = tshift ? tshift[l] : nullptr;
        s1.mix_row[0] = 0; s1.mix_row[1] = 2; s1.mix_row[2] = 3;
        if (first) {
            s1.has_emb = 1; s1.emb = make_view(m.emb); s1.token = out.token; s1.ln0_w = m.ln0_w; s1.ln0_b = m.ln0_b;
            s1.x_out = xa;
        } else {
            s1.src = cur;
            s1.x_out = cur.n_parts ? xa : nullptr;
        }
        const float* x_now = (first || cur.n_parts) ? xa : cur.resid;     // the assembled row after this stage
        first = false;
        for (int k = 0; k < 3; ++k) s1.y[k] = rkv + static_cast<size_t>(k) * D;
        // LoRA branches in the order w, a, g, v (v absent on layer 0)
        const rwkvq_qtensor* t1[4] = {&L.w1, &L.a1, &L.g1, &L.v1};
        const rwkvq_qtensor* t2[4] = {&L.w2, &L.a2, &L.g2, &L.v2};
        const int mixrow[4] = {1, 4, 5, 3}, acts[4] = {1, 0, 2, 0};
        const int n_lora = layer0 ? 3 : 4;
        Op s2{};
        s2.type = OP_TMIX;
        int off = 0;
        for (int b = 0; b < n_lora; ++b) {
            rc = validate_qtensor(t1[b], "rwkvq_decoder(lora down)");
            if (rc) return rc;
            rc = validate_qtensor(t2[b], "rwkvq_decoder(lora up)");
            if (rc) return rc;
            RWKVQ_REQUIRE(t1[b]->rows == D && t1[b]->cols == t2[b]->rows && t2[b]->cols == D, RWKVQ_E_SHAPE,
                          "rwkvq_decoder: LoRA branch %d has shapes [%d,%d] x [%d,%d]", b, t1[b]->rows, t1[b]->cols,
                          t2[b]->rows, t2[b]->cols);
            s1.l[b] = make_view(*t1[b]); s2.l[b] = make_view(*t2[b]);
            s1.lora_mix_row[b] = mixrow[b]; s1.lora_off[b] = s2.lora_off[b] = off;
            s1.lora_act[b] = s2.lora_act[b] = acts[b];
            off += (t1[b]->cols + 3) / 4 * 4;
        }
        RWKVQ_REQUIRE(off <= kPMaxRank, RWKVQ_E_LIMIT, "rwkvq_decoder: LoRA ranks sum to %d, at most %d", off, kPMaxRank);
        {
            // LoRA-down units on the CTAs the r/k/v GEMVs leave idle: column groups of 32, and as
            // many row chunks (at most 8: the consumer adds them in one batch of loads) as fit
            const int cg = (off + 31) / 32, spare = grid - s1.n_units;
            RWKVQ_REQUIRE(spare >= cg, RWKVQ_E_LIMIT, "rwkvq_decoder: %d CTAs left for %d LoRA column groups", spare, cg);
            int chunks = spare / cg;
            if (chunks > 8) chunks = 8;
            const int rows = ((D + chunks - 1) / chunks + 31) / 32 * 32;
            chunks = (D + rows - 1) / rows;
            s1.lora_cg = cg; s1.lora_rows = rows; s1.lora_chunks = s2.lora_chunks = chunks;
        }
        {
            // LoRA-up slots of 64 rows, every branch padded to whole slots
            int slot = 0;
            for (int b = 0; b < n_lora; ++b) {
                RWKVQ_REQUIRE(lora_mode_host(*t2[b]) < 2 && t2[b]->cols % 16 == 0 && aligned(t2[b]->codes, 16) &&
                                  lora_mode_host(*t1[b]) < 3,
                              RWKVQ_E_DTYPE, "rwkvq_decoder: LoRA up matrix %d is not 8-bit asym / per-row int8", b);
                s2.off64[b] = slot * 64;
                for (int r = 0; r < (t2[b]->rows + 63) / 64; ++r) {
                    RWKVQ_REQUIRE(slot < kUpSlots, RWKVQ_E_LIMIT, "rwkvq_decoder: LoRA ranks need more than %d slots of 64 rows", kUpSlots);
                    s2.slot_br[slot++] = b;
                }
            }
            s2.up_slots = slot;
        }
        s1.n_lora = s2.n_lora = n_lora;
        s1.lora_stride = s2.lora_stride = off; s1.lora_part = s2.lora_part = lora_part;
        {
            const int tm = static_cast<int>(tmix_smem_bytes(s2.up_slots, s2.lora_chunks, off));
            const int ld = (s1.lora_rows / 32) * 4 * kPThreads * 4;         // LoRA-down staging words
            if (tm > work) work = tm;
            if (ld > work) work = ld;
            if (32 * 32 * 4 > work) work = 32 * 32 * 4;
        }
        need_work(s1);
        out.ops.push_back(s1);
        // ---- S2: time-mix core
        s2.D = D; s2.H = H; s2.layer0 = layer0 ? 1 : 0;
        s2.r = rkv; s2.k = rkv + D; s2.v = rkv + 2 * static_cast<size_t>(D);
        s2.w0 = L.w0; s2.a0 = L.a0; s2.v0 = L.v0; s2.k_k = L.k_k; s2.k_a = L.k_a; s2.r_k = L.r_k;
        s2.lnx_w = L.lnx_w; s2.lnx_b = L.lnx_b; s2.v_first = v_first; s2.state = wkv ? wkv[l] : nullptr; s2.og = og;
        out.ops.push_back(s2);
        // ---- S3: output projection + residual -> the other buffer
        Op s3{};
        const rwkvq_qtensor* wo[1] = {&L.Wo};
        rc = gemv_op(s3, wo, 1, grid, false, "output projection");
        if (rc) return rc;
        RWKVQ_REQUIRE(s3.rows == D && s3.cols == D, RWKVQ_E_SHAPE, "rwkvq_decoder: output projection must be [%d, %d]", D, D);
        float* x_next = (x_now == xa) ? xb : xa;
        s3.in_kind = IN_VEC; s3.D = D; s3.src.resid = og;
        s3.epilogue = RWKVQ_EPI_ADD; s3.resid_out = x_now; s3.y[0] = x_next;
        need_work(s3);
        out.ops.push_back(s3);
        // ---- S4: ffn key
        Op s4{};
        const rwkvq_qtensor* wfk[1] = {&L.Wfk};
        rc = gemv_op(s4, wfk, 1, grid, false, "ffn key");
        if (rc) return rc;
        RWKVQ_REQUIRE(s4.rows == F && s4.cols == D, RWKVQ_E_SHAPE, "rwkvq_decoder: ffn key must be [%d, %d]", F, D);
        s4.in_kind = IN_LN; s4.D = D; s4.src.resid = x_next;
        s4.ln_w = L.ln2_w; s4.ln_b = L.ln2_b; s4.mix = L.ffn_x_k; s4.shift = cshift ? cshift[l] : nullptr;
        s4.epilogue = RWKVQ_EPI_RELU2; s4.y[0] = hffn;
        need_work(s4);
        out.ops.push_back(s4);
        // ---- S5: ffn value; with a K split the partial sums join the residual row in the next prologue
        Op s5{};
        const rwkvq_qtensor* wfv[1] = {&L.Wfv};
        rc = gemv_op(s5, wfv, 1, grid, true, "ffn value");
        if (rc) return rc;
        RWKVQ_REQUIRE(s5.rows == D && s5.cols == F, RWKVQ_E_SHAPE, "rwkvq_decoder: ffn value must be [%d, %d]", D, F);
        s5.in_kind = IN_VEC; s5.D = D; s5.src.resid = hffn;
        cur = VecSrc{};
        if (s5.ks > 1) {
            s5.part_out = part;
            cur.resid = x_next; cur.part = part; cur.n_parts = s5.ks; cur.stride = s5.rows_padded;
        } else {
            float* x_after = (x_next == xa) ? xb : xa;
            s5.epilogue = RWKVQ_EPI_ADD; s5.resid_out = x_next; s5.y[0] = x_after;
            cur.resid = x_after;
        }
        need_work(s5);
        out.ops.push_back(s5);
    }
    // ---- head on LN_out of the final row, then the argmax
    Op hd{};
    const rwkvq_qtensor* ht[1] = {&m.head};
    rc = gemv_op(hd, ht, 1, grid, false, "head");
    if (rc) return rc;
    RWKVQ_REQUIRE(hd.rows == V && hd.cols == D, RWKVQ_E_SHAPE, "rwkvq_decoder: head must be [%d, %d]", V, D);
    hd.in_kind = IN_LN; hd.D = D; hd.src = cur; hd.ln_w = m.lnout_w; hd.ln_b = m.lnout_b;
    hd.y[0] = logits;
    need_work(hd);
    out.ops.push_back(hd);
    Op a1{};
    a1.type = OP_ARGMAX_PART; a1.V = V; a1.logits = logits; a1.pv = pv; a1.pi = pi;
    out.ops.push_back(a1);
    Op a2 = a1;
    a2.type = OP_ARGMAX_FINAL; a2.token_feed = out.token;
    out.ops.push_back(a2);
    out.work_bytes = (work + 15) / 16 * 16;
    return RWKVQ_OK;
}

int smem_bytes(int work_bytes, int D) {
    return static_cast<int>(2 * sizeof(Op)) + work_bytes + 2 * D * static_cast<int>(sizeof(float)) +
           (256 + 32) * static_cast<int>(sizeof(float)) + 16;
}

// Resident CTAs of the persistent kernel: 2 per SM (fewer if shared memory does not allow it).
int resident_grid(int smem, int* grid) {
    int dev = 0, sms = 0, per_sm = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess && smem > 48 * 1024)
        e = cudaFuncSetAttribute(decode_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_persist_kernel, kPThreads, smem);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_decoder: occupancy query: %s", cudaGetErrorString(e));
    if (per_sm < 1) return fail(RWKVQ_E_LIMIT, "rwkvq_decoder: %d bytes of shared memory do not fit an SM", smem);
    *grid = sms * (per_sm > 2 ? 2 : per_sm);
    return RWKVQ_OK;
}

// The program depends on the grid (work split) and the grid on the shared memory the
// program needs: plan for 2 CTAs per SM, then check that the kernel is really that resident.
int plan(const rwkvq_model& m, float* const* wkv, float* const* ts, float* const* cs, void* base, float* logits,
         Built& b, int* grid, int* smem) {
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_decoder: %s", cudaGetErrorString(e));
    int g = 2 * sms;
    for (int attempt = 0; attempt < 2; ++attempt) {
        int rc = build_program(m, wkv, ts, cs, g, base, logits, b);
        if (rc) return rc;
        *smem = smem_bytes(b.work_bytes, m.n_embd);
        int real = 0;
        rc = resident_grid(*smem, &real);
        if (rc) return rc;
        if (real == g) { *grid = g; return RWKVQ_OK; }
        g = real;
    }
    return fail(RWKVQ_E_LIMIT, "rwkvq_decoder: could not settle the resident grid");
}

}  // namespace

extern "C" {

size_t rwkvq_decoder_workspace_bytes(const rwkvq_model* m) {
    if (!m || !m->layers) return 0;
    Built b;
    int grid = 0, smem = 0;
    if (plan(*m, nullptr, nullptr, nullptr, nullptr, nullptr, b, &grid, &smem)) return 0;
    return b.bytes;
}

int rwkvq_decoder_create(const rwkvq_model* m, float* const* wkv, float* const* tshift, float* const* cshift,
                         void* workspace, size_t workspace_bytes, float* logits, void* stream, rwkvq_decoder** out) {
    RWKVQ_REQUIRE(m && m->layers && wkv && tshift && cshift && workspace && out, RWKVQ_E_NULL,
                  "rwkvq_decoder_create: null pointer");
    RWKVQ_REQUIRE(aligned(workspace, 256), RWKVQ_E_ALIGN, "rwkvq_decoder_create: workspace must be 256-byte aligned");
    Built b;
    int grid = 0, smem = 0;
    int rc = plan(*m, wkv, tshift, cshift, workspace, logits, b, &grid, &smem);
    if (rc) return rc;
    RWKVQ_REQUIRE(workspace_bytes >= b.bytes, RWKVQ_E_LIMIT, "rwkvq_decoder_create: workspace %zu < %zu bytes",
                  workspace_bytes, b.bytes);
    int coop = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    RWKVQ_REQUIRE(coop != 0, RWKVQ_E_ARCH, "rwkvq_decoder_create: device does not support cooperative launches");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the barrier words start at zero; the program is copied from pageable memory (the copy
    // has left the host buffer when cudaMemcpyAsync returns)
    cudaError_t e = cudaMemsetAsync(b.sync, 0, 64 * sizeof(unsigned int), s);
    if (e == cudaSuccess) e = cudaMemsetAsync(b.token, 0, sizeof(long long), s);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(b.ops_dev, b.ops.data(), b.ops.size() * sizeof(Op), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_decoder_create: %s", cudaGetErrorString(e));
    rwkvq_decoder* d = new rwkvq_decoder();
    d->n_ops = static_cast<int>(b.ops.size()); d->grid = grid; d->smem = smem; d->work_bytes = b.work_bytes;
    d->D = m->n_embd; d->V = m->vocab_size;
    d->ops_dev = b.ops_dev; d->sync = b.sync; d->token = b.token; d->logits = b.logits;
    d->trace = nullptr;
    *out = d;
    return RWKVQ_OK;
}

void rwkvq_decoder_destroy(rwkvq_decoder* d) { delete d; }

int64_t* rwkvq_decoder_token(rwkvq_decoder* d) { return d ? reinterpret_cast<int64_t*>(d->token) : nullptr; }
float* rwkvq_decoder_logits(rwkvq_decoder* d) { return d ? d->logits : nullptr; }
int rwkvq_decoder_grid(const rwkvq_decoder* d) { return d ? d->grid : 0; }
int rwkvq_decoder_stages(const rwkvq_decoder* d) { return d ? d->n_ops : 0; }
void rwkvq_decoder_set_trace(rwkvq_decoder* d, void* buf) { if (d) d->trace = static_cast<unsigned long long*>(buf); }

int rwkvq_decoder_step(rwkvq_decoder* d, void* stream) {
    RWKVQ_REQUIRE(d != nullptr, RWKVQ_E_NULL, "rwkvq_decoder_step: decoder is null");
    PersistArgs a{d->ops_dev, d->n_ops, d->sync, d->work_bytes, d->D, d->trace};
    void* args[1] = {&a};
    cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(decode_persist_kernel), dim3(d->grid),
                                                dim3(kPThreads), args, static_cast<size_t>(d->smem),
                                                static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_decoder_step: %s", cudaGetErrorString(e));
    return RWKVQ_OK;
}

int rwkvq_decoder_status(rwkvq_decoder* d, void* stream) {
    RWKVQ_REQUIRE(d != nullptr, RWKVQ_E_NULL, "rwkvq_decoder_status: decoder is null");
    int st = 0;
    cudaError_t e = cudaMemcpyAsync(&st, d->sync + 2, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_decoder_status: %s", cudaGetErrorString(e));
    if (st != 0) return fail(st, "rwkvq_decoder: a grid barrier of the persistent kernel ran out of polls");
    return RWKVQ_OK;
}

}  // extern "C"
