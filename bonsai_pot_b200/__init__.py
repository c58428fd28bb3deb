"""B200 (sm_100a) attention hot path for bonsai-pot: KV-cache quantise-and-write,
Q norm + RoPE, split-KV decode attention and batched-prefill causal attention
over the reference's Q8_0 cache layout, behind the C ABI of
include/bonsai_attn.h."""
from .errors import (ConfigError, ContextOverflow, CudaError, DeviceLost, DeviceTimeout, PotError,  # noqa: F401
                     PrefillTooLarge)
from .attention import AttnContext  # noqa: F401
from .kv_snapshot import KvSnapshot  # noqa: F401
from .errors import IoError  # noqa: F401
from .model import GenerateOptions, Model, Sampler, Session, StopReason  # noqa: F401

__all__ = ["AttnContext", "KvSnapshot", "PotError", "ConfigError", "ContextOverflow", "PrefillTooLarge",
           "DeviceLost", "CudaError", "DeviceTimeout", "IoError", "Model", "Session", "Sampler", "GenerateOptions", "StopReason"]
