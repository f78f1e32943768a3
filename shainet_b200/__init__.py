"""B200 (sm_100a) attention path for SHAInet's LLaMA/Qwen decoder block.

The product is ``lib/libshainet_attn.so`` (C ABI in ``include/shainet_attn.h``);
this package is its host-side mirror of the reference's ``LlamaBlock`` attention
interface and, around it, of the Q8_0 weights, the whole block and the token loop.  Importing does not load the library; the first use does, and fails
loudly if it has not been built."""
from . import sharding  # noqa: F401
from .attention import (AttnContext, Decoder, KVCache, LlamaAttention, LlamaBlock, Q8Weight, ShainetAttnError, default_scale, device_count,  # noqa: F401
                        forward_batched_dev, F_GENERIC, F_SPLITK, F_TENSOR, F_UNFUSED, F_INPUTS_READY, F_TICKET_MERGE, F_TENSOR_1CTA)
