"""B200-native NVFP4 attention (SageAttention3 path): thin PyTorch front end over ``libsage3_b200.so``."""
from .api import (sageattn, sageattn3_blackwell, sageattn4_blackwell, pack_kv, sageattn_varlen, sageattn_from_host, quantize_qkv, fp4_attention,
                  QuantizedQKV, buffer_sizes)

__all__ = ["sageattn", "sageattn3_blackwell", "sageattn4_blackwell", "pack_kv", "sageattn_varlen", "sageattn_from_host", "quantize_qkv", "fp4_attention",
           "QuantizedQKV", "buffer_sizes"]
