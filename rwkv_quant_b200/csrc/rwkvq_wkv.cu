// WKV-7 recurrence and the time-mix tail.
//
// State S[dv][dk] (64 x 64 fp32 per batch element and head).  Per step
//     sa = S a;   S = S diag(w) + sa b^T + v k^T;   y = S r
// (call site backends/metal/quant_model.py:118-125, math models/rwkv7_ref.py:244-254,
// prototype kernel tests/bench_wkv_shared.py:64-97).  The 64 state rows are
// independent, so a CTA owns one (batch, head) and its threads keep tiles of the state in
// registers for the whole scan; the two dot products per step end in shuffles.  The
// r/w/k/v/a/b rows of following steps are staged in shared memory ahead of time (see below).
#include "rwkvq_common.cuh"

namespace rwkvq {

constexpr int kS = 64;             // head size

struct WkvArgs {
    const float *r, *w, *k, *v, *a, *b;   // [B, T, H, 64]
    const float* h_in;                     // [B, H, 64, 64] or null (zeros)
    float* out;                            // [B, T, H, 64]
    float* h_out;                          // [B, H, 64, 64] (may alias h_in)
    int B, T, H;
};

// Thread tile.  What bounds a step is the shared-memory return path (128 bytes per clock and SM:
// every float a thread loads costs its warp one cycle, broadcast or not), so a thread owns a
// tile of R state rows x 8 columns: per step it loads 8 columns of a, w, k, b, r and R values of v
// (40 + R floats for 8 R state elements; one row x 16 columns would load 81 for 16).  Eight lanes
// span the 64 columns of a row group, so a dot product ends in three shuffle stages; a warp holds
// four row groups.  R = 8: 64 threads, least shared-memory traffic per step, for full grids;
// R = 4, and R = 2 with 4 CTAs per head: shorter steps for grids that leave SMs empty (measured:
// two CTAs of 128 threads per head were slower than one of R = 4).
//
// Staging: the r/w/k/v/a/b rows of kWkvChunk steps form one chunk; a ring of kWkvStages chunks in
// shared memory is filled with 16-byte cp.async copies issued two chunks (16 steps) ahead, so a load
// from HBM has thousands of cycles to land.  Within a chunk the warps run free of one another,
// and the CTA meets at one barrier per chunk, which also releases the ring slot that is refilled next.
constexpr int kWkvChunk = 8;
constexpr int kWkvStages = 3;
constexpr int kWkvStepFloats = 6 * kS;                            // a, w, k, b, r, v
constexpr int kWkvChunkFloats = kWkvChunk * kWkvStepFloats;
constexpr size_t kWkvSmemBytes = sizeof(float) * kWkvStages * kWkvChunkFloats;

__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gmem_src) {
    const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Sums y[0..R) over the 8 lanes of a row group, one shuffle stage per call (m = 1, 2, 4), halving
// the number of live values at each stage (a lane keeps the half its lane bit selects and sends
// the other); afterwards y[0] is the total of row `row` - lanes 0..R-1 of the group end with
// distinct rows.
template <int R>
struct RowReduce {
    int n = R, row = 0;
    __device__ __forceinline__ void stage(float (&y)[R], int c, int m) {
        if (n > 1) {
            const int half = n >> 1;
            const bool up = (c & m) != 0;
#pragma unroll
            for (int i = 0; i < R / 2; ++i) {
                if (i < half) {
                    const float send = up ? y[i] : y[i + half];
                    const float keep = up ? y[i + half] : y[i];
                    y[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, m);
                }
            }
            row += up ? half : 0;
            n = half;
        } else {
            y[0] += __shfl_xor_sync(0xFFFFFFFFu, y[0], m);
        }
    }
};

// SPLIT CTAs share one (batch, head): the state rows are independent, so CTA s of the group owns
// rows s * 64 / SPLIT .. and reads the same staged r/w/k/v/a/b rows (small grids are bound by the
// latency of a step, which shrinks with the work a warp has per step).
template <int R, int SPLIT>
__global__ void __launch_bounds__(512 / R / SPLIT, 4) wkv7_kernel(const WkvArgs p) {
    constexpr int kThreads = 512 / R / SPLIT;
    extern __shared__ __align__(16) float ring[];
    const int bh = blockIdx.x / SPLIT, bi = bh / p.H, hi = bh % p.H;
    const int tid = threadIdx.x, c = tid & 7, dv0 = (blockIdx.x % SPLIT) * (kS / SPLIT) + (tid >> 3) * R;
    float2 h[R][4];                               // rows dv0 + j, columns 8c + 2q, 8c + 2q + 1
    const size_t hbase = (static_cast<size_t>(bh) * kS + dv0) * kS + c * 8;
#pragma unroll
    for (int j = 0; j < R; ++j) {
        if (p.h_in) {
            const float4 lo4 = *reinterpret_cast<const float4*>(p.h_in + hbase + j * kS);
            const float4 hi4 = *reinterpret_cast<const float4*>(p.h_in + hbase + j * kS + 4);
            h[j][0] = make_float2(lo4.x, lo4.y); h[j][1] = make_float2(lo4.z, lo4.w);
            h[j][2] = make_float2(hi4.x, hi4.y); h[j][3] = make_float2(hi4.z, hi4.w);
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) h[j][q] = make_float2(0.f, 0.f);
        }
    }
    const size_t row0 = (static_cast<size_t>(bi) * p.T * p.H + hi) * kS;     // step 0 of this (batch, head)
    const size_t step_stride = static_cast<size_t>(p.H) * kS;
    // Copy roles: a step is 96 pieces of 16 bytes (row q >> 4 of a, w, k, b, r, v; floats 4 (q & 15) ..).
    // R = 4: thread q < 96 copies piece q of every step; R = 8: thread q < 48 copies pieces q and q + 48.
    constexpr int kOwn = kThreads >= 96 ? 1 : 2, kCopiers = 96 / kOwn;
    const float* cp_src[kOwn];
#pragma unroll
    for (int o = 0; o < kOwn; ++o) {
        const int q = (tid + o * kCopiers) % 96, row = q >> 4;
        const float* base = row == 0 ? p.a : row == 1 ? p.w : row == 2 ? p.k : row == 3 ? p.b : row == 4 ? p.r : p.v;
        cp_src[o] = base + row0 + (q & 15) * 4;
    }
    auto issue = [&](int chunk) {
        if (tid >= kCopiers) return;
        float* stage = ring + (chunk % kWkvStages) * kWkvChunkFloats + tid * 4;
        const int t0 = chunk * kWkvChunk;
#pragma unroll
        for (int s = 0; s < kWkvChunk; ++s) {
            if (t0 + s < p.T) {
#pragma unroll
                for (int o = 0; o < kOwn; ++o)
                    cp_async16(stage + s * kWkvStepFloats + o * kCopiers * 4, cp_src[o] + (t0 + s) * step_stride);
            }
        }
    };
    // One step of the recurrence on the rows staged at `st`.  Packed fp32 arithmetic: two lanes per
    // instruction, each lane an IEEE fma (measured 13 % faster at B = 16 than the same step in scalar
    // instructions, which also need 237 registers instead of 198).
    // The output sums of step t are reduced and stored during step t+1, stage by stage beside the
    // shuffles of that step's S a, so that only one shuffle chain per step is exposed.
    float yp[R];                                      // per-lane partial sums of the pending output
    int tp = -1;                                      // its step (-1: none yet)
#pragma unroll
    for (int j = 0; j < R; ++j) yp[j] = 0.f;
    auto step = [&](int t, const float* st) {
        float2 x[4], kv[4];
        auto load8 = [&](int row, float2 (&d)[4]) {
            const float4 lo4 = *reinterpret_cast<const float4*>(st + row * kS + c * 8);
            const float4 hi4 = *reinterpret_cast<const float4*>(st + row * kS + c * 8 + 4);
            d[0] = make_float2(lo4.x, lo4.y); d[1] = make_float2(lo4.z, lo4.w);
            d[2] = make_float2(hi4.x, hi4.y); d[3] = make_float2(hi4.z, hi4.w);
        };
        float vv[R];
#pragma unroll
        for (int j = 0; j < R; j += 2) {
            const float2 v2 = *reinterpret_cast<const float2*>(st + 5 * kS + dv0 + j);
            vv[j] = v2.x; vv[j + 1] = v2.y;
        }
        load8(0, x);                                  // a
        float sa[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
            float2 p0 = __fmul2_rn(h[j][0], x[0]), p1 = __fmul2_rn(h[j][1], x[1]);
            p0 = __ffma2_rn(h[j][2], x[2], p0);
            p1 = __ffma2_rn(h[j][3], x[3], p1);
            p0 = __fadd2_rn(p0, p1);
            sa[j] = p0.x + p0.y;
        }
        RowReduce<R> rr;
#pragma unroll
        for (int m = 1; m < 8; m <<= 1) {
#pragma unroll
            for (int j = 0; j < R; ++j) sa[j] += __shfl_xor_sync(0xFFFFFFFFu, sa[j], m);
            rr.stage(yp, c, m);
        }
        if (tp >= 0 && c < R) p.out[row0 + tp * step_stride + dv0 + rr.row] = yp[0];
        load8(3, x);                                  // b
        load8(2, kv);                                 // k
        float2 u[R][4];                               // v k^T + sa b^T
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const float2 sa2 = make_float2(sa[j], sa[j]), vv2 = make_float2(vv[j], vv[j]);
#pragma unroll
            for (int q = 0; q < 4; ++q) u[j][q] = __ffma2_rn(vv2, kv[q], __fmul2_rn(sa2, x[q]));
        }
        load8(1, x);                                  // w
        load8(4, kv);                                 // r
#pragma unroll
        for (int j = 0; j < R; ++j) {
#pragma unroll
            for (int q = 0; q < 4; ++q) h[j][q] = __ffma2_rn(x[q], h[j][q], u[j][q]);
            float2 p0 = __fmul2_rn(h[j][0], kv[0]), p1 = __fmul2_rn(h[j][1], kv[1]);
            p0 = __ffma2_rn(h[j][2], kv[2], p0);
            p1 = __ffma2_rn(h[j][3], kv[3], p1);
            p0 = __fadd2_rn(p0, p1);
            yp[j] = p0.x + p0.y;
        }
        tp = t;
    };
    const int n_chunks = (p.T + kWkvChunk - 1) / kWkvChunk;
#pragma unroll
    for (int ch = 0; ch < kWkvStages - 1; ++ch) {
        if (ch < n_chunks) issue(ch);
        cp_async_commit();                       // empty groups keep the count uniform
    }
    for (int ch = 0; ch < n_chunks; ++ch) {
        cp_async_wait<kWkvStages - 2>();         // this thread's pieces of chunk ch have landed
        __syncthreads();                         // everybody's have, and chunk ch-1 is consumed
        if (ch + kWkvStages - 1 < n_chunks) issue(ch + kWkvStages - 1);     // into the slot of chunk ch-1
        cp_async_commit();
        const float* stage = ring + (ch % kWkvStages) * kWkvChunkFloats;
        const int t0 = ch * kWkvChunk, n = min(kWkvChunk, p.T - t0);
        if (n == kWkvChunk) {
#pragma unroll
            for (int s = 0; s < kWkvChunk; ++s) step(t0 + s, stage + s * kWkvStepFloats);
        } else {
            for (int s = 0; s < n; ++s) step(t0 + s, stage + s * kWkvStepFloats);
        }
    }
    cp_async_wait<0>();
    {                                                 // the output of the last step
        RowReduce<R> rr;
#pragma unroll
        for (int m = 1; m < 8; m <<= 1) rr.stage(yp, c, m);
        if (tp >= 0 && c < R) p.out[row0 + tp * step_stride + dv0 + rr.row] = yp[0];
    }
#pragma unroll
    for (int j = 0; j < R; ++j) {
        *reinterpret_cast<float4*>(p.h_out + hbase + j * kS) = make_float4(h[j][0].x, h[j][0].y, h[j][1].x, h[j][1].y);
        *reinterpret_cast<float4*>(p.h_out + hbase + j * kS + 4) = make_float4(h[j][2].x, h[j][2].y, h[j][3].x, h[j][3].y);
    }
}

// (group_norm(wkv) * ln_w + ln_b + (sum r*k*r_k) * v) * g per (row, head); a warp per
// pair, two-pass variance as in backends/metal/fused_tail.py:43-76.
__global__ void __launch_bounds__(128) wkv_tail_kernel(const float* wkv, const float* r, const float* k,
                                                       const float* v, const float* r_k, const float* ln_w,
                                                       const float* ln_b, const float* g, float* out,
                                                       int n_pairs, int H, float eps) {
    const int pair = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= n_pairs) return;
    const int hd = pair % H;
    const size_t base = static_cast<size_t>(pair) * kS;
    const int hb = hd * kS;
    const float x0 = wkv[base + lane], x1 = wkv[base + lane + 32];
    float s = x0 + x1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    const float mean = s / kS;
    const float d0 = x0 - mean, d1 = x1 - mean;
    float s2 = d0 * d0 + d1 * d1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s2 += __shfl_xor_sync(0xFFFFFFFFu, s2, o);
    const float inv = 1.0f / sqrtf(s2 / kS + eps);
    float dp = r[base + lane] * k[base + lane] * r_k[hb + lane] +
               r[base + lane + 32] * k[base + lane + 32] * r_k[hb + lane + 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dp += __shfl_xor_sync(0xFFFFFFFFu, dp, o);
    out[base + lane] = (d0 * inv * ln_w[hb + lane] + ln_b[hb + lane] + dp * v[base + lane]) * g[base + lane];
    out[base + lane + 32] =
        (d1 * inv * ln_w[hb + lane + 32] + ln_b[hb + lane + 32] + dp * v[base + lane + 32]) * g[base + lane + 32];
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

int rwkvq_wkv7(const float* r, const float* w, const float* k, const float* v, const float* a,
               const float* b, const float* h_in, float* out, float* h_out, int B, int T, int H,
               int head_size, void* stream) {
    RWKVQ_REQUIRE(r && w && k && v && a && b && out && h_out, RWKVQ_E_NULL, "rwkvq_wkv7: null pointer");
    RWKVQ_REQUIRE(head_size == kS, RWKVQ_E_SHAPE, "rwkvq_wkv7: head size %d, only 64 is built", head_size);
    RWKVQ_REQUIRE(B >= 1 && T >= 1 && H >= 1, RWKVQ_E_SHAPE, "rwkvq_wkv7: B=%d T=%d H=%d", B, T, H);
    RWKVQ_REQUIRE(aligned(h_out, 16) && aligned(h_in, 16), RWKVQ_E_ALIGN, "rwkvq_wkv7: state must be 16-byte aligned");
    RWKVQ_REQUIRE(aligned(r, 16) && aligned(w, 16) && aligned(k, 16) && aligned(v, 16) && aligned(a, 16) && aligned(b, 16),
                  RWKVQ_E_ALIGN, "rwkvq_wkv7: r/w/k/v/a/b must be 16-byte aligned");
    WkvArgs p{r, w, k, v, a, b, h_in, out, h_out, B, T, H};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // few (batch, head) pairs: smaller tiles and several CTAs per pair, so that a step is short;
    // full grids: the largest tile (least shared-memory traffic and issue per state element)
    const int pairs = B * H;
    if (pairs > 2 * 148) wkv7_kernel<8, 1><<<pairs, 64, kWkvSmemBytes, st>>>(p);
    else if (pairs > 74) wkv7_kernel<4, 1><<<pairs, 128, kWkvSmemBytes, st>>>(p);
    else wkv7_kernel<2, 4><<<pairs * 4, 64, kWkvSmemBytes, st>>>(p);
    return check_launch("rwkvq_wkv7");
}

int rwkvq_wkv_tail(const float* wkv, const float* r, const float* k, const float* v, const float* r_k,
                   const float* ln_w, const float* ln_b, const float* g, float* out, int N, int H,
                   int head_size, float eps, void* stream) {
    RWKVQ_REQUIRE(wkv && r && k && v && r_k && ln_w && ln_b && g && out, RWKVQ_E_NULL, "rwkvq_wkv_tail: null pointer");
    RWKVQ_REQUIRE(head_size == kS, RWKVQ_E_SHAPE, "rwkvq_wkv_tail: head size %d, only 64 is built", head_size);
    RWKVQ_REQUIRE(N >= 1 && H >= 1, RWKVQ_E_SHAPE, "rwkvq_wkv_tail: N=%d H=%d", N, H);
    const int pairs = N * H;
    wkv_tail_kernel<<<(pairs + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(wkv, r, k, v, r_k, ln_w, ln_b, g,
                                                                                  out, pairs, H, eps);
    return check_launch("rwkvq_wkv_tail");
}

}  // extern "C"
