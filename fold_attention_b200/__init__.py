"""fold_attention_b200: FoldAttention's two hot paths, built for B200 (sm_100a).

Softmax attention whose cross-CTA reductions do not depend on the order work
runs in: a deterministic attention backward (integer-grid dQ, private dK/dV)
and a quantised paged-KV decode whose split partials combine by plain
addition. The public names and signatures are the reference's
(src/fold_attention/__init__.py:11-16); all device work runs in
libfold_b200.so through a C ABI. There is no CPU or PyTorch fallback.
"""

from .interface import fold_attn_func, fold_attn_varlen_func, fold_attn_with_kvcache
from .kv_cache import FoldKVCache

__version__ = "0.1.0"

__all__ = ["FoldKVCache", "fold_attn_func", "fold_attn_varlen_func", "fold_attn_with_kvcache"]
