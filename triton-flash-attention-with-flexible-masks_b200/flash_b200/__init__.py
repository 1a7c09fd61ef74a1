"""B200-native flash attention with document masks; mirrors the reference's `flash_triton` module."""
from .host import attention_host, bind_to_gpu_numa_node
from .ops import (SCORE_FUNC_MODE0_NOPE, SCORE_FUNC_MODE1_DOC, FlashAttention, attention, check_status,
                  debug_mask, maybe_contiguous)

__all__ = ["SCORE_FUNC_MODE0_NOPE", "SCORE_FUNC_MODE1_DOC", "FlashAttention", "attention", "attention_host", "bind_to_gpu_numa_node", "check_status",
           "debug_mask", "maybe_contiguous"]
