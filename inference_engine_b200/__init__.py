"""B200-native int8 KV-cache attention path (quantize-on-write + split-K paged decode attention
+ chunked-prefill attention) behind the call signatures of kbwal/inference-engine's
qwen3-1.7b/kernels.py.  `inference_engine_b200.kernels` is the drop-in module."""
from . import kernels  # noqa: F401
from .kernels import (  # noqa: F401
    LayerKVCache,
    decode_attention,
    dequantize_kv_prefix,
    fused_norm_rope_prefill,
    fused_rope_kv_decode,
    make_layer_cache,
    prefill_attention,
    quantize_kv_prefill,
)
