from . import attention, block, delta, embedding, feedforward, fused, gated_attention, latent, linear_attention, mlstm, norms, positions, scan  # noqa: F401  (registration)
from .registry import FAMILIES, part_class, register_part, unregister_part
from .block import Block
from .runtime import Branch, HostBatch, Runtime, StepContext

__all__ = ["FAMILIES", "part_class", "register_part", "unregister_part", "Block", "Branch", "HostBatch", "Runtime", "StepContext"]
