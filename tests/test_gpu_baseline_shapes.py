"""The linear shapes of the benchmark configurations at their full sizes, batch 1 / 8 / 64:
  * one RWKV-7 1.5B layer in the `reduction` layouts (sym@8 projections [2048,2048], sym@6 channel
    mix [8192,2048] and [2048,8192], per-row int8 LoRA g1 / g2, asym LoRA w1 / w2) and the
    `compression` layouts (sb6@5 projections, sb6@4 channel mix; the [8192,2048] sb6@4 matrix with
    fp16 activations is the single-GEMV configuration);
  * reference = fp64 product with the device-side dequantisation, which the golden tests pin bit
    for bit to the codec; tolerance rel-max <= 1e-3 (measured ~1e-6);
  * batch-size independence: row n of a batched GEMV call equals the same row computed alone, bit
    for bit; the tensor-core GEMM used beyond 2 rows is held to the same 1e-3.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-3

SHAPES = [
    ("sym", 8, 2048, 2048), ("sym", 6, 8192, 2048), ("sym", 6, 2048, 8192),
    ("sb6", 5, 2048, 2048), ("sb6", 4, 8192, 2048), ("sb6", 4, 2048, 8192),
]


def _lin(layout, bits, rows, cols, seed):
    from rwkv_quant_b200 import synth
    from rwkv_quant_b200.backends.cuda import linear_for
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * 0.02
    fn = {"sb6": synth.quant_sb6, "sym": synth.quant_sym, "rtn": synth.quant_rtn, "asym": synth.quant_asym}[layout]
    return linear_for(fn("w", "g", w, bits))


@pytest.mark.parametrize("layout,bits,rows,cols", SHAPES)
def test_layer_linear_shapes_batches(cuda_lib, layout, bits, rows, cols):
    lin = _lin(layout, bits, rows, cols, seed=rows * 7 + cols + bits)
    w64 = lin._dequant_w(torch.float32).double()
    g = torch.Generator().manual_seed(99)
    x64 = torch.randn(64, cols, generator=g).cuda()
    outs = {}
    for n in (1, 8, 64):
        for dt in (torch.float32, torch.float16):
            x = x64[:n].to(dt)
            y = lin(x)
            ref = x.double() @ w64.t()
            err = (y.double() - ref).abs().max().item() / ref.abs().max().item()
            assert y.shape == (n, rows) and err <= TOL, (layout, bits, n, dt, err)
            if dt == torch.float32:
                outs[n] = y
    # beyond 2 rows the operator reads the weights once for the whole batch (fp16 operands on the
    # tensor cores): rows agree with the exact single-vector kernel within the operand rounding
    scale = outs[1].abs().max().item()
    assert (outs[8][:1] - outs[1]).abs().max().item() <= 5e-4 * scale
    assert (outs[64][:8] - outs[8]).abs().max().item() <= 5e-4 * scale
    # the tensor-core GEMM (what the model uses beyond 2 rows): fp16 activations scaled per token
    from rwkv_quant_b200.backends.cuda import ops
    x512 = torch.randn(512, cols, generator=g).cuda()           # at and beyond 128 rows the operator itself
    y = lin(x512)                                               # switches to the GEMM, as the reference does
    ref = x512.double() @ w64.t()
    assert (y.double() - ref).abs().max().item() <= TOL * ref.abs().max().item(), (layout, bits, 512)
    for n in (8, 64):
        y = ops.gemm(lin.dq, x64[:n], check=True)
        ref = x64[:n].double() @ w64.t()
        err = (y.double() - ref).abs().max().item() / ref.abs().max().item()
        assert err <= TOL, (layout, bits, n, "gemm", err)


def test_lora_shapes(cuda_lib):
    """LoRA pairs of a 1.5B layer in file orientation [in, out]: asym@6 g64 (w: 2048x96, 96x2048)
    and per-row int8 (g: 2048x256, 256x2048), 1 and 8 rows."""
    from rwkv_quant_b200 import synth
    from rwkv_quant_b200.backends.cuda import ops
    g = torch.Generator().manual_seed(5)
    for layout, bits, rin, rout in (("asym", 6, 2048, 96), ("asym", 6, 96, 2048), ("rtn", 8, 2048, 256), ("rtn", 8, 256, 2048)):
        w = torch.randn(rin, rout, generator=g) * 0.05
        fn = synth.quant_asym if layout == "asym" else synth.quant_rtn
        dq = ops.DeviceQT(fn("w", "g", w, bits))
        wd = dq.dequant(torch.float32, True).half().double()            # the loader's precision
        for n in (1, 8):
            x = torch.randn(n, rin, generator=g).cuda()
            y = ops.gemv_t(dq.bufs, dq.meta, x, 0, True)
            ref = x.double() @ wd
            assert (y.double() - ref).abs().max().item() <= TOL * ref.abs().max().item(), (layout, rin, rout, n)
