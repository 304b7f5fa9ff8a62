"""B200-native (sm_100a) inference backend for ``.rwkvq`` RWKV-7 checkpoints.

Layout of the package
  formats/        ``.rwkvq`` container reader / writer, checkpoint dataclasses
  synth.py        seeded random-init builds packed in the file layouts
  csrc/           CUDA kernels and the C-ABI (``include/rwkvq_b200.h``)
  backends/cuda/  the reference's backend operator surface on top of the C-ABI
"""
__version__ = "0.1.0"
