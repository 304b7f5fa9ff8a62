"""``.rwkvq`` container and checkpoint dataclasses."""
from .container import (FORMAT, FORMAT_VERSION, QuantizedCheckpoint,  # noqa: F401
                        QuantizedTensor, is_raw_lora_world, load_raw,
                        open_rwkvq, save_rwkvq)
