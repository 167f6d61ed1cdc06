"""The operator namespace: the nine names of the reference's ``native_sparse_attention.ops``, plus the two steps its layer
leaves to other code (sliding-window attention, the gated sum of the branches, rotary embedding)."""
from .compress import avgpool_compress, linear_compress, weightedpool_compress
from .compressed_attention import compressed_attention
from .decode import compressed_attention_decode, flash_attention_decode, topk_sparse_attention_decode
from .flash_attention import flash_attention_varlen
from .gate_combine import gate_combine
from .rope import rope
from .sliding_window import sliding_window_attention
from .topk_sparse_attention import topk_sparse_attention
from .utils import get_compressed_seqlens

__all__ = [
    "avgpool_compress",
    "weightedpool_compress",
    "linear_compress",
    "flash_attention_varlen",
    "sliding_window_attention",
    "gate_combine",
    "rope",
    "compressed_attention",
    "topk_sparse_attention",
    "flash_attention_decode",
    "compressed_attention_decode",
    "topk_sparse_attention_decode",
    "get_compressed_seqlens",
]
