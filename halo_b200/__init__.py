"""halo_b200: a Blackwell-native LLM / MoE training framework.

Process-wide defaults that must be in place before torch or transformers are imported live here,
as in the reference's package init (halo/__init__.py).
"""

import os as _os

_os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
_os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "8")
_os.environ.setdefault("TORCH_NCCL_AVOID_RECORD_STREAMS", "1")

__version__ = "0.1.0"
