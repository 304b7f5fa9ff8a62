"""CPU oracle for the quantized RWKV-7 forward path.

TEST INFRASTRUCTURE ONLY. Nothing under ``rwkv_quant_b200/`` imports this
package; it is used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline / reference legs of ``bench.py`` as the checker and as the timed
CPU baseline, never as a compute fallback.

Contents
  codec_np   numpy restatement of the ``.rwkvq`` bit layouts and the four
             dequantisers (follows rwkv_quant/formats/codec.py)
  model_np   stateful fp32 forward (follows
             rwkv_quant/backends/metal/quant_model.py and
             rwkv_quant/models/rwkv7_ref.py)
  wkv7_seq.c sequential-order WKV-7 recurrence in plain C (follows the
             prototype kernel in tests/bench_wkv_shared.py)
  quant_np   numpy restatement of the sb6 and sym block quantizers (follows
             rwkv_quant/calibration/groupwise.py)
  wkv7_chunked_np  the same recurrence advanced a chunk of tokens at a time
             (derivation of a chunked scan; checked against model_np.wkv7_np)
"""
