/*
 * rwkvq_b200.h -- C ABI of librwkvq_b200.so: sm_100a kernels for the quantized
 * RWKV-7 forward path of `.rwkvq` checkpoints.
 *
 * The reference project has no FFI: its backend boundary is a set of Python
 * classes in rwkv_quant/backends/metal/ that launch Metal kernels.  Each entry
 * point below names the reference operator it stands behind (paths relative to
 * the reference project root).  The Python classes in
 * rwkv_quant_b200/backends/cuda/ bind these symbols through ctypes and expose
 * the reference's class / function names on top of them.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller, unless the
 *     parameter name ends in `_host`;
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it
 *     and nothing synchronises;
 *   - no entry point allocates or frees device memory;
 *   - return value: 0 on success, a negative RWKVQ_E_* code otherwise
 *     (rwkvq_strerror() gives the text, rwkvq_last_error_detail() the detail of
 *     the calling thread's last failure);
 *   - thread-safe when called on distinct streams (calls that share a stream must come
 *     from one thread at a time, as for any stream-ordered API); rwkvq_gemv_static is the
 *     exception documented at its declaration.
 */
#ifndef RWKVQ_B200_H
#define RWKVQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RWKVQ_OK          0
#define RWKVQ_E_SHAPE    -1   /* a dimension violates a layout rule (IN % 256, ...)   */
#define RWKVQ_E_ALIGN    -2   /* a pointer is not aligned as the kernel needs          */
#define RWKVQ_E_DTYPE    -3   /* unsupported dtype / layout / bit width                */
#define RWKVQ_E_ARCH     -4   /* device is not sm_100                                  */
#define RWKVQ_E_LAUNCH   -5   /* the CUDA runtime refused the launch                   */
#define RWKVQ_E_TIMEOUT  -6   /* a bounded device-side wait ran out                    */
#define RWKVQ_E_NULL     -7   /* a required pointer is null                            */
#define RWKVQ_E_LIMIT    -8   /* a size exceeds a documented maximum                   */
#define RWKVQ_E_FORMAT   -9   /* a file is not a readable .rwkvq container             */

/* element types of activation / output buffers */
#define RWKVQ_F32   0
#define RWKVQ_F16   1
#define RWKVQ_BF16  2

/* tensor layouts ("kind" in the .rwkvq manifest; formats/codec.py:28-41) */
#define RWKVQ_KIND_DENSE 0    /* bf16 as stored                                         */
#define RWKVQ_KIND_SB6   1    /* block 32, super-block 8, 6-bit scale/min codes         */
#define RWKVQ_KIND_SYM   2    /* block 16, super-block 16, int8 scale code, no min      */
#define RWKVQ_KIND_ASYM  3    /* block gs, fp32 scale/min per block, uint8 codes        */
#define RWKVQ_KIND_RTN   4    /* per-row fp16 scale, int8 codes or biased nibbles       */

/* epilogues of the GEMV family */
#define RWKVQ_EPI_NONE      0   /* y = W x                                             */
#define RWKVQ_EPI_RELU2     1   /* y = relu(W x)^2      (cmix key, quant_model.py:800) */
#define RWKVQ_EPI_ADD       2   /* y = resid + W x      (residual add of a block)      */

/*
 * One quantized tensor in the FILE layout (no repack).  rows/cols are the stored
 * shape; for linear weights rows = OUT, cols = IN.  Unused pointers are NULL.
 * Field <-> file buffer (formats/schema.py:45-81):
 *   codes   sb6/sym@6: codes_packed u8 [rows, cols/2];  sym@8/rtn@8: codes i8
 *           [rows, cols];  asym: codes u8 [rows, cols];  rtn@<=4: codes_packed u8
 *           [rows, ceil(cols/2)];  dense: bf16 [rows, cols]
 *   qh,qh2  gw_qh / gw_qh2 u8 [rows, cols/8]
 *   qsqm    gw_qsqm u8 [rows, cols/256, 12]              (sb6)
 *   qs      gw_qs  i8 [rows, cols/16]                    (sym)
 *   d,dm    gw_d / gw_dm f16 [rows, cols/256]
 *   scale   asym: gw_scale f32 [rows, ceil(cols/gs)];  rtn: scale f16 [rows]
 *   mn      asym: gw_min  f32 [rows, ceil(cols/gs)]
 */
typedef struct rwkvq_qtensor {
    int32_t kind;
    int32_t bits;
    int32_t rows;
    int32_t cols;
    int32_t gs;
    int32_t sb;
    const void* codes;
    const void* qh;
    const void* qh2;
    const void* qsqm;
    const void* qs;
    const void* d;
    const void* dm;
    const void* scale;
    const void* mn;
    /* Optional device-side relayout of the small side streams (same byte count as
     * the file buffers, made once at load by rwkvq_relayout_*; codes stay as in the
     * file).  When both are NULL the kernels read the file buffers only.
     *   dev_meta    sb6: [rows, cols/256] records of 16 B: word t = the scale/min codes of
     *               blocks 2t, 2t+1 and one byte of (d | dm << 16)
     *   dev_planes  bit-planes regrouped per block so that one shift + mask yields
     *               the high code bits of 4 weights (see rwkvq_relayout_planes) */
    const void* dev_meta;
    const void* dev_planes;
} rwkvq_qtensor;

const char* rwkvq_strerror(int code);
const char* rwkvq_last_error_detail(void);
/* 0 when the current device is compute capability 10.x, RWKVQ_E_ARCH otherwise */
int rwkvq_check_device(void);
int rwkvq_abi_version(void);

/*
 * Dequantise a tensor to a dense [rows, cols] buffer.
 * Stands behind codec.dequant_{sb6,sym,asym,rtn} (formats/codec.py:183-292) and
 * the Metal dequant kernel SymQuantLinear._dequant_w
 * (backends/metal/quant_linear_sym.py:275-363, 433-452).
 * out_dtype RWKVQ_F32 is bit-exact against the numpy codec (separate multiply
 * and add, fp16 round-trip of the block scale / min); F16 / BF16 round that
 * value once.  `round_bf16` != 0 rounds the fp32 value to bf16 first (what
 * reader._dequantize_one does, formats/reader.py:114-127) before the cast.
 */
int rwkvq_dequant(const rwkvq_qtensor* t, void* out, int out_dtype, int round_bf16,
                  void* stream);

/*
 * Quantized matrix-vector product for N right-hand sides, weights streamed in
 * the file layout and never materialised:  y[n, o] = epi( sum_c W[o, c] x[n, c] ).
 * Stands behind GwQuantLinear.__call__ / _gemv1 / _gemv_nb
 * (backends/metal/quant_linear_gw.py:842-940), SymQuantLinear._gemv
 * (quant_linear_sym.py:498-516) and QuantLinearV2.__call__
 * (quant_linear_v2.py:322-351).
 *   x      [N, ldx] of x_dtype, y [N, ldy] fp32, resid [N, ldy] fp32 (EPI_ADD)
 * fp32 accumulation.  Layout rules: sb6 / sym need cols % 256 == 0; the other
 * kinds are unrestricted (a slower generic kernel serves ragged shapes).
 */
int rwkvq_gemv(const rwkvq_qtensor* t, const void* x, int x_dtype, int N, int64_t ldx,
               float* y, int64_t ldy, int epilogue, const float* resid, void* stream);

/*
 * Sparse outlier overrides of a per-row tensor, applied to a product over its packed codes:
 *   y[n, r] = epi( y[n, r] + sum_{j in row r} delta[j] * x[n, cols[j]] ),  delta = override - quantized value.
 * Stands behind the CSR tail of the reference's per-row kernels (backends/metal/quant_linear_v2.py:47-55,
 * CSR build quant_linear.py:17; formats/codec.py:279-292 defines the override).  row_ptr [rows + 1], cols and
 * delta [n_overrides] sorted by (row, column); call rwkvq_gemv with RWKVQ_EPI_NONE first, the epilogue belongs here.
 */
int rwkvq_outlier_tail(const int32_t* row_ptr, const int32_t* cols, const float* delta, int rows, const void* x,
                       int x_dtype, int N, int64_t ldx, float* y, int64_t ldy, int epilogue, const float* resid, void* stream);

/*
 * Block quantizer for the sb6 layout on the device.  Stands behind the reference's host-side search
 * quantizer (calibration/groupwise.py:207-300 `_gw_one` with 8 blocks of 32 per super-block, as called by
 * formats/writer.py:236-269 `_make_qt_gw_sb6` for the modes asym_sb6 / asym_sb6_search / asym_sb6_aw).
 *   w [rows, ldw] fp32 on the device, cols a multiple of 256; bits 4, 5 or 6;
 *   search != 0: the 8-factor scale search with least-squares refit per block (asym_sb6_search);
 *   ex2 (optional, [cols] fp32): E[x^2] of the input channels, weights of the search criterion (asym_sb6_aw).
 * Outputs (device): q [rows, cols] codes 0 .. 2^bits - 1, qs [rows, cols/32] scale codes 1 .. 63,
 * qm [rows, cols/32] min codes -31 .. 31, d / dm [rows, cols/256] fp16 super-scales: the `parts` of the
 * reference, which its packers (and rwkv_quant_b200.quantize) turn into the file buffers.
 * Arithmetic as in the reference (fp32, IEEE division, round-half-to-even); sums over a block run in a
 * different order than torch's, so a code can differ where a quotient sits on a rounding boundary.
 */
int rwkvq_quantize_sb6(const float* w, int64_t ldw, int rows, int cols, int bits, int search, const float* ex2,
                       uint8_t* q, uint8_t* qs, int8_t* qm, void* d, void* dm, void* stream);

/*
 * The same for the symmetric layout (blocks of 16, int8 block-scale codes against one fp16 per 256 weights);
 * stands behind calibration/groupwise.py:358-473 `_sym_one` as called by formats/writer.py `_make_qt_gw_sym`
 * (modes sym, sym_aw, sym_plain; outlier fractions are not supported, as in the reference's packed path).
 *   bits 6 or 8; factors [n_factors] fp32 on the device: the scale factors of the search — the reference's
 *   19 float32 nodes of torch.linspace(0.7, 1.15, 19), or {1.0} for the plain mode; ex2 as above.
 * Outputs (device): q [rows, cols] signed codes, qs [rows, cols/16] int8 scale codes, d [rows, cols/256] fp16.
 */
int rwkvq_quantize_sym(const float* w, int64_t ldw, int rows, int cols, int bits, const float* factors, int n_factors,
                       const float* ex2, int8_t* q, int8_t* qs, void* d, void* stream);

/*
 * The same product for a SMALL BATCH of right-hand sides (decode streams, short verify runs)
 * with every packed weight byte read once for the whole batch.  Stands behind the multi-column
 * GEMV kernels of the reference, which decode each weight once for up to 4 columns and loop
 * over chunks of 4 (GwQuantLinear._gemv_nb / _get_kernel_k3nb, backends/metal/quant_linear_gw.py:
 * 658-744, 850-905; SymQuantLinear._gemv, quant_linear_sym.py:485-516): here one pass serves
 * up to 16 columns per CTA (the token groups of a larger batch run side by side in one launch).
 *   x [N, ldx] fp32 (rows 16-byte aligned, ldx % 4 == 0), y / resid [N, ldy] fp32.
 *   Tensors: sb6 with dev_meta (and dev_planes at 5 / 6 bits), sym (dev_planes at 6 bits),
 *   per-row int8 with cols % 128 == 0; RWKVQ_E_DTYPE otherwise (use rwkvq_gemv).
 * Arithmetic: fp16 tensor-core products with BOTH operands carried as two fp16 terms (weights:
 * q*s as rounded product + its exact rounding error, block mins on the per-block sums of the
 * activations; activations: hi + lo of x scaled per token by a power of two chosen from its max|x|),
 * fp32 accumulation: the result agrees with an fp32 dequantise-and-multiply, and with rwkvq_gemv,
 * to ~1e-6 of max|y| (a column's last bits may depend on the batch it is computed in; two calls on
 * the same input give the same bits).  The K split is reduced across a thread-block cluster through
 * distributed shared memory: no scratch for partial sums.
 * With RWKVQ_BATCH_FAST=1 in the environment (read once per process) single fp16 operands are used
 * instead (weights fp16(q*s+m)): ~25 % faster at 32 rows and more, results within ~3e-4 of max|y|
 * per call (the precision of rwkvq_gemm), and sb6 / sym tensors with more than 32 rows run on the
 * tcgen05 tensor cores (rows of 128 as the UMMA M, the batch as its N, accumulator in tensor memory).
 *   workspace: rwkvq_gemv_batch_workspace_bytes(N) bytes, 16-byte aligned: a status word (first
 *   int32: RWKVQ_E_TIMEOUT if a bounded wait on the tensor-core pipeline ran out; read it after
 *   synchronising the stream, 0 = ok) and one float per row, the max|x| a one-block-per-row
 *   pre-pass writes before the product kernel starts.
 */
size_t rwkvq_gemv_batch_workspace_bytes(int N);
int rwkvq_gemv_batch(const rwkvq_qtensor* t, const float* x, int N, int64_t ldx, float* y, int64_t ldy,
                     int epilogue, const float* resid, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Quantized linear for MANY right-hand sides on the tcgen05 tensor cores (prefill,
 * batched decode):  y[n, o] = epi( sum_c W[o, c] x[n, c] ),  n < M.
 * Stands behind the N >= 128 branch of GwQuantLinear.__call__ / SymQuantLinear.__call__
 * (backends/metal/quant_linear_gw.py:846-849, quant_linear_sym.py:481-484: dequantise to
 * fp16, then a dense matmul) with the dequantisation fused into the operand producer, so
 * no dense copy of W is ever written.  Operands are fp16 (weights: fp16(q*s+m); tokens:
 * scaled per row by a power of two), accumulation fp32 in tensor memory.
 *   x [M, ldx] fp32, y [M, ldy] fp32, sb6 / sym tensors only.
 *   workspace: rwkvq_gemm_workspace_bytes_for(M, IN) bytes, 256-byte aligned (or
 *   rwkvq_gemm_workspace_bytes(M), which covers IN <= 16384); it holds the fp16 copy of x the
 *   TMA loads read, the split-K accumulator tiles and a header.  Its first int32 is a status word the
 *   kernel sets to RWKVQ_E_TIMEOUT if a bounded wait on the tensor-core pipeline ran out
 *   (read it after synchronising the stream; 0 = ok).
 */
size_t rwkvq_gemm_workspace_bytes(int M);
size_t rwkvq_gemm_workspace_bytes_for(int M, int max_cols);
int rwkvq_gemm(const rwkvq_qtensor* t, const float* x, int M, int64_t ldx, float* y, int64_t ldy,
               int epilogue, const float* resid, void* workspace, size_t workspace_bytes, void* stream);
/* The same product on activations the caller has already brought into the form the kernel reads
 * (rwkvq_seq_ln_shift_mix_prep writes it): x16 fp16 [M, rwkvq_gemm_x16_pitch(IN)] = x * row_scale[m],
 * row_scale [M] fp32 powers of two.  The workspace (same size rule) then only carries the header
 * and the split-K tiles. */
size_t rwkvq_gemm_x16_pitch(int cols);
int rwkvq_gemm_x16(const rwkvq_qtensor* t, const void* x16, const float* row_scale, int M, float* y, int64_t ldy,
                   int epilogue, const float* resid, void* workspace, size_t workspace_bytes, void* stream);

/*
 * K same-shape matrices, K different inputs, one launch: y[k] = W_k x[k].
 * Stands behind GwQuantLinearFused / SymQuantLinearFused
 * (quant_linear_gw.py:943-1020, quant_linear_sym.py:519-574); results are
 * bit-identical to K separate rwkvq_gemv calls with N = 1.
 *   ts [K] host array of tensors (same kind, bits, rows, cols)
 *   x  [K, cols] of x_dtype, y [K, rows] fp32
 */
int rwkvq_gemv_fused(const rwkvq_qtensor* ts_host, int K, const void* x, int x_dtype,
                     float* y, void* stream);

/*
 * Matrix-vector product against a tensor stored [in, out] (world-naming LoRA
 * matrices, formats/codec.py:514-535):  y[n, o] = act( sum_i x[n, i] Wt[i, o] ).
 * Stands behind the dense LoRA matmuls of QuantTMix._lora
 * (backends/metal/quant_model.py:462-526, _mm :204-208) with the weights read
 * from the file bytes instead of an fp16 copy.  `round_w` != 0 applies the
 * reference's load-time rounding fp16(bf16(w)) to every weight
 * (quant_model.py:128-154).  act: 0 none, 1 tanh, 2 sigmoid.
 */
int rwkvq_gemv_t(const rwkvq_qtensor* t, const float* x, int N, int64_t ldx,
                 float* y, int64_t ldy, int act, int round_w, void* stream);

/*
 * Up to four LoRA branches for N rows in two launches on the tensor cores:
 *   y_i[n, :] = act_i( x_i[n, :] @ W1_i ) @ W2_i,   W1_i stored [D, r_i], W2_i stored [r_i, C]
 * (C = D, or any multiple of 32 shared by all branches: a column range of the up projections, as a
 * head-sharded model holds; y_i is [N, C] contiguous)
 * Stands behind QuantTMix._lora for every row count above 2 (backends/metal/quant_model.py:462-526:
 * the decay, in-context rate, gate and value-residual branches; dense fp16 matmuls there).  The
 * matrices are read from their file bytes (asym / per-row int8 / dense bf16) and used in the
 * loader's precision fp16(bf16(w)), which is exact in fp16; x and the rank-space activations enter
 * as fp16 pairs hi + lo (~2^-22 relative), accumulation fp32.  act: 0 none, 1 tanh, 2 sigmoid.
 *   t1_host / t2_host  host arrays of n_br descriptors; xs_host / ys_host host arrays of n_br device
 *   pointers to [N, D] (x) and [N, C] (y) fp32 rows (contiguous, 16-byte aligned); acts_host host array.
 *   Requirements: D % 128 == 0, ranks multiples of 16 up to 512 (RWKVQ_E_SHAPE otherwise: use
 *   rwkvq_gemv_t).  workspace: rwkvq_lora_pair_workspace_bytes(N, max rank) bytes, 16-byte aligned.
 */
size_t rwkvq_lora_pair_workspace_bytes(int N, int max_rank);
int rwkvq_lora_pair(const rwkvq_qtensor* t1_host, const rwkvq_qtensor* t2_host, int n_br, const float* const* xs_host,
                    float* const* ys_host, const int* acts_host, int N, int D, void* workspace, size_t workspace_bytes,
                    void* stream);

/*
 * Single-vector rwkvq_gemv that allocates nothing.  NO COUNTERPART IN THE
 * REFERENCE: added for callers that may not allocate on the call path (an
 * inference server's steady-state loop that has frozen its memory pool, a host
 * thread under a real-time budget, code running where cudaMalloc would
 * synchronise the device).
 *   y[o] = epi( sum_c W[o, c] x[c] ),  x [cols] of x_dtype, y / resid [rows] fp32.
 * The K loop is split across CTAs; the slices' partial sums and arrival counters
 * live in a 260 KiB __device__ array inside the library, whose address is looked
 * up once per device.  The call issues one cudaMemsetAsync (counters) and one
 * kernel on `stream`; it calls no cudaMalloc / cudaFree nor any allocating
 * library routine.
 *   limits  rows <= 4096, cols <= 16384 (RWKVQ_E_LIMIT beyond); sb6 tensors need
 *           dev_meta (and dev_planes at 5 / 6 bits), sym@6 needs dev_planes, per-row
 *           int8 needs cols % 128 == 0 (RWKVQ_E_DTYPE otherwise); x 16-byte aligned.
 *   set-up  the first call on a device resolves the array's address (and may load
 *           the module): make it before any stream capture begins.
 *   races   every call on a device uses the same array: two calls that can
 *           overlap (different streams or threads) race on it; serialise them.
 * Results equal rwkvq_gemv's up to fp32 summation order and are bit-identical
 * from call to call.
 */
int rwkvq_gemv_static(const rwkvq_qtensor* t, const void* x, int x_dtype, float* y,
                      int epilogue, const float* resid, void* stream);


/*
 * WKV-7 recurrence with state in and out, any T >= 1, head size 64:
 *   sa = S a;  S = S diag(w) + sa b^T + v k^T;  y = S r      (S indexed [value, key])
 * Stands behind wkv7_infer(r, w, k, v, a, b, state) -> (out, new_state) of the
 * external rwkv_metal package as called at backends/metal/quant_model.py:118-125
 * (math: models/rwkv7_ref.py:244-254).  r..b [B, T, H, 64] fp32 (w is the decay),
 * h_in [B, H, 64, 64] or NULL for a zero state, h_out may alias h_in.
 */
int rwkvq_wkv7(const float* r, const float* w, const float* k, const float* v, const float* a,
               const float* b, const float* h_in, float* out, float* h_out, int B, int T, int H,
               int head_size, void* stream);

/*
 * (group_norm(wkv) * ln_w + ln_b + (sum_head r*k*r_k) * v) * g for N rows of H heads.
 * Stands behind fused_tail.wkv_tail (backends/metal/fused_tail.py:92-110).
 */
int rwkvq_wkv_tail(const float* wkv, const float* r, const float* k, const float* v, const float* r_k,
                   const float* ln_w, const float* ln_b, const float* g, float* out, int N, int H,
                   int head_size, float eps, void* stream);

/*
 * Glue of the sequence (prefill) path for all B*T tokens of a call; the single-token forms
 * live inside rwkvq_decode_step.
 *   rwkvq_seq_ln_shift_mix  xn = LayerNorm(x[b,t]); prev = xn[b,t-1] (t = 0: shift_in[b] or
 *       zeros when NULL); out[m][b,t] = xn + (prev - xn) * mix[m] for m < n_mix (1 or 6);
 *       shift_out[b] = xn[b,T-1].  Stands behind _layer_norm + _token_shift_stateful + the lerp
 *       stack (quant_model.py:281-301, 648-651, 803-806).  x [B,T,D], out [n_mix,B,T,D] fp32.
 *   rwkvq_seq_tmix_pre  decay, gates, kk, k and v updates feeding the WKV-7 scan
 *       (quant_model.py:700-712): w = exp(-0.606531 sigmoid(yw + w0)), a = sigmoid(ya + a0),
 *       kk = l2norm per head of k * k_k, k2 = k (1 + (a - 1) k_a),
 *       v2 = v + (v_first - v) sigmoid(yv + v0) (yv, v_first, v0 NULL on layer 0: v2 = v),
 *       neg_kk = -kk, kk_a = kk * a.  All [n_tokens, H * 64] fp32.
 */
int rwkvq_seq_ln_shift_mix(const float* x, const float* ln_w, const float* ln_b, const float* shift_in,
                           const float* mix, int n_mix, float* out, float* shift_out, int B, int T, int D,
                           void* stream);
/* rwkvq_seq_ln_shift_mix with each mix row written in the form(s) its consumers read, selected
 * per mix by modes[m] (host array; bit 0: scaled fp16 copy + scale for rwkvq_gemm_x16 into
 * out_x16[m] [N, D + 64] / out_scale[m] [N]; bit 1: fp16 hi/lo split as rwkvq_split_fp16 into
 * out_split[m] [N, 2 D]; bit 2: fp32 row into out_f32[m] [N, D]).  Pointer tables are host arrays
 * of n_mix device pointers (entries of unselected forms are ignored).  D even. */
int rwkvq_seq_ln_shift_mix_prep(const float* x, const float* ln_w, const float* ln_b, const float* shift_in,
                                const float* mix, int n_mix, const int* modes, void* const* out_x16,
                                float* const* out_scale, void* const* out_split, float* const* out_f32,
                                float* shift_out, int B, int T, int D, void* stream);
/* x fp32 [rows, cols] -> out fp16 [rows, 2 * cols] = [fp16(x) | fp16(x - fp16(x))]: the operand of the
 * dense LoRA products of long sequences (x @ W = [hi | lo] @ [W; W] on fp16 tensor cores, fp32
 * accumulation; the reference casts x to fp16 there: quant_model.py:204-208). */
int rwkvq_split_fp16(const float* x, void* out_fp16, int64_t rows, int cols, void* stream);
/* Rows of the embedding table for n_tokens ids in the loader's precision fp16(bf16(.)), LayerNorm 0
 * applied: x [n_tokens, D] fp32 (quant_model.py:853, 975-976; ids are clamped to the table).  And a
 * plain LayerNorm of n_rows rows (eps 1e-5), the final norm of the sequence path (:281). */
int rwkvq_seq_embed_ln0(const rwkvq_qtensor* emb, const int64_t* tokens, const float* ln_w, const float* ln_b, float* x,
                        int64_t n_tokens, int D, void* stream);
int rwkvq_seq_layer_norm(const float* x, const float* ln_w, const float* ln_b, float* out, int64_t n_rows, int D, void* stream);
int rwkvq_seq_tmix_pre(const float* k, const float* v, const float* yw, const float* ya, const float* yv,
                       const float* v_first, const float* w0, const float* a0, const float* v0,
                       const float* k_k, const float* k_a, float* w, float* k2, float* v2, float* neg_kk,
                       float* kk_a, int64_t n_tokens, int H, void* stream);

/* One layer / one model as device pointers; dense vectors are fp32 [D] already in the
 * reference's load-time precision (quant_model.py:128-154). LoRA tensors are stored [in, out]. */
typedef struct rwkvq_layer {
    const float *ln1_w, *ln1_b, *ln2_w, *ln2_b;
    const float* x_mix;                 /* [6, D]: r, w, k, v, a, g lerp coefficients */
    const float *w0, *a0, *v0;          /* [D]; v0 NULL on layer 0 */
    const float *k_k, *k_a, *r_k, *lnx_w, *lnx_b;
    const float* ffn_x_k;
    rwkvq_qtensor w1, w2, a1, a2, v1, v2, g1, g2;
    rwkvq_qtensor Wr, Wk, Wv, Wo, Wfk, Wfv;
} rwkvq_layer;

typedef struct rwkvq_model {
    int32_t n_layer, n_embd, head_size, vocab_size, ffn_dim, max_rank;
    rwkvq_qtensor emb, head;
    const float *ln0_w, *ln0_b, *lnout_w, *lnout_b;
    const rwkvq_layer* layers;          /* HOST array [n_layer] */
} rwkvq_model;

/* Bytes of device scratch rwkvq_decode_step needs for batch B (logits included).
 * The workspace must be zero-filled once before its first use (arrival counters of
 * the K-split GEMV live in it and reset themselves after every launch). */
size_t rwkvq_decode_workspace_bytes(const rwkvq_model* m_host, int B);

/*
 * One token for B independent streams: embedding gather, all layers, head.
 * Stands behind QuantRWKV7.forward_stateful with T = 1
 * (backends/metal/quant_model.py:964-990; block :827-836, time-mix :638-728,
 * channel-mix :803-809).  State is updated in place:
 *   wkv_host[l]    [B, H, 64, 64]   tshift_host[l], cshift_host[l]  [B, D]
 * (host arrays of device pointers; a fresh stream starts from zeros).
 * logits [B, vocab] fp32 (NULL: kept in the workspace), next_tokens [B] int64 greedy
 * argmax (NULL: skipped), tokens [B] int64 on the device.
 * Linears: B = 1 the single-vector tensor-core GEMV; 3 <= B <= 256 the weights-once small-batch
 * kernels in two-term precision (see rwkvq_gemv_batch), of which r / k / v, the ffn key and the head
 * take the tcgen05 form at 33-48 streams and r / k / v and the head at 49-64 (RWKVQ_TCB_EXACT=0 / 1 in
 * the environment, read once: none / all three at every B above 32); RWKVQ_BATCH_FAST=1 selects single
 * fp16 operands instead; larger B the prefill GEMM.
 */
int rwkvq_decode_step(const rwkvq_model* m_host, int B, const int64_t* tokens,
                      float* const* wkv_host, float* const* tshift_host, float* const* cshift_host,
                      void* workspace, size_t workspace_bytes, float* logits, int64_t* next_tokens,
                      void* stream);

/*
 * Load-time relayout of the side streams of an sb6 / sym tensor for the decode
 * kernels; pure byte / bit permutations, no value changes, same total size.
 * No counterpart in the reference's file format; it plays the role of the Metal
 * loader's K3 interleave (formats/codec.py:390-435) without growing the data.
 *   meta    out [rows, cols/256, 16] u8           (sb6 only)
 *   planes  out u32: sb6@5 [rows, cols/32]; sb6@6 [rows, cols/32, 2];
 *           sym@6 [rows, cols/16]                 (not needed at 4 / 8 bits)
 */
int rwkvq_relayout_meta(const rwkvq_qtensor* t, void* meta_out, void* stream);
int rwkvq_relayout_planes(const rwkvq_qtensor* t, void* planes_out, void* stream);

/*
 * Tensor-parallel row split (2.9B variant): every rank computes the output rows it owns
 * with rwkvq_gemv on a row slice of the tensor (any row range is a valid tensor in every
 * layout: the file buffers slice on axis 0, cf. formats/reader.py:144-152) and the slices
 * are exchanged by peer stores over NVLink.  No counterpart in the reference (single
 * device); the exchange stands where an NCCL all-gather would.
 *
 *   rwkvq_tp_alloc / rwkvq_tp_free   zero-filled device buffer from cudaMalloc (set-up time
 *       only), shareable with rwkvq_ipc_export
 *   rwkvq_ipc_export / _open / _close  64-byte CUDA IPC handle of a buffer; mapping of a
 *       peer's buffer into this process (peer access enabled lazily)
 *   rwkvq_tp_allgather_store   src [count] fp32 = this rank's slice.  Stores it into
 *       segment `rank` of dst_ptrs[p] for every rank p (host array of `world` device
 *       pointers, entry `rank` being this rank's own buffer), raises flag_ptrs[p][rank] =
 *       epoch, and waits until flag_ptrs[rank][0..world) all reached the epoch = the number
 *       of this exchange, kept in `epoch_ctr` (device, [world] words, zero at start, private
 *       to the rank), so a captured CUDA graph can be replayed; every rank must issue the
 *       same sequence of exchanges; use two destination buffers alternately per site.  After `max_spins` polls the kernel gives up, stores
 *       RWKVQ_E_TIMEOUT in *status (device int, 0 = ok) and returns; count % 4 == 0.
 */
int rwkvq_tp_alloc(size_t bytes, void** out);
int rwkvq_tp_free(void* p);
int rwkvq_ipc_export(const void* dev_ptr, void* handle64);
int rwkvq_ipc_open(const void* handle64, void** out);
int rwkvq_ipc_close(void* p);
int rwkvq_tp_allgather_store(const float* src, int count, float* const* dst_ptrs,
                             unsigned int* const* flag_ptrs, int rank, int world, unsigned int* epoch_ctr,
                             int* status, long long max_spins, void* stream);

/*
 * Torch-free reader of the .rwkvq container (host side): the C counterpart of
 * codec.open_rwkvq / reader.load_raw (formats/codec.py:496-511, formats/reader.py:42-93).
 *   rwkvq_file_open     maps the file read-only, parses the safetensors header and the manifest;
 *                       RWKVQ_E_FORMAT for a foreign container, a missing manifest, a
 *                       format_version above 2, or buffers that do not fit the file
 *   rwkvq_file_tensor   descriptor with HOST pointers into the mapping (valid until close);
 *                       rows = product of the leading dimensions, cols = the last one;
 *                       `transposed` = stored [in, out]; sparse overrides (int32 [n, 2] row/column,
 *                       bf16 [n] values) when the tensor carries them, else NULL / 0
 *   rwkvq_file_upload   one device allocation holding the tensor's buffers (256-byte aligned each),
 *                       filled by cudaMemcpyAsync on `stream`; dev_view is what the kernels take
 *                       (dev_meta / dev_planes NULL: run rwkvq_relayout_* for the decode layouts);
 *                       release with rwkvq_file_free_slab
 */
typedef struct rwkvq_file rwkvq_file;
typedef struct rwkvq_file_info {
    int32_t format_version;
    int32_t naming;                 /* 0 = world, 1 = custom */
    int32_t n_layer, n_embd, head_size, vocab_size;
    int32_t n_tensors;
} rwkvq_file_info;
int rwkvq_file_open(const char* path, rwkvq_file** out);
void rwkvq_file_close(rwkvq_file* f);
int rwkvq_file_get_info(const rwkvq_file* f, rwkvq_file_info* out);
const char* rwkvq_file_tensor_key(const rwkvq_file* f, int index);
int rwkvq_file_tensor(const rwkvq_file* f, const char* key, rwkvq_qtensor* host_view, int32_t* transposed,
                      const void** outlier_indices, const void** outlier_values, int64_t* n_outliers);
int rwkvq_file_upload(const rwkvq_file* f, const char* key, rwkvq_qtensor* dev_view, void** slab, void* stream);
int rwkvq_file_free_slab(void* slab);

#ifdef __cplusplus
}
#endif
#endif /* RWKVQ_B200_H */
