"""B200 (sm_100a) Native Sparse Attention kernels behind the reference project's entry points.

    from nsa_from_scratch_b200 import nsa_forward, NSAConfig

All arithmetic runs in hand-written CUDA kernels reached through the C ABI of
libnsa_b200.so (include/nsa_b200.h); there is no CPU or torch fallback."""
from .config import NSAConfig
from .compressed import compressed_attention
from .selected import selected_attention
from .sliding import sliding_attention
from .gating import combine
from .forward import nsa_forward, nsa_forward_fp8, _resolve_block_indices
from .backward import selected_backward
from .fp8 import quantize_to_fp8, selected_attention_fp8
from .native import selected_attention_cuda, selected_backward_cuda
from .host import nsa_forward_host
from .layer import NSAAttention, nsa_attention_token_major, rope_cache
from .graph import GraphedForward
from .decode import KVCache, nsa_decode, GraphedDecoder
from .scoring import compressed_block_scores, select_blocks_compressed
from .moba import moba_attention

__all__ = [
    "NSAConfig", "compressed_attention", "selected_attention", "sliding_attention", "combine", "nsa_forward",
    "nsa_forward_fp8", "nsa_forward_host", "selected_backward", "quantize_to_fp8", "selected_attention_fp8",
    "selected_attention_cuda", "selected_backward_cuda", "NSAAttention", "nsa_attention_token_major", "rope_cache",
    "GraphedForward", "KVCache", "nsa_decode", "GraphedDecoder", "compressed_block_scores", "select_blocks_compressed",
    "moba_attention",
]
