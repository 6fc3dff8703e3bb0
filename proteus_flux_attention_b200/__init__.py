"""B200-native ASPA attention: the reference package's public names on sm_100a kernels."""
from .aspa import (AdaptiveSparseAttention, AdaptiveSparseAttentionBlock, AdaptiveSparseProtoAttention, MLP,
                   ModelConfig)
from .chunked_shortlist import (ChunkedShortlistConfig, ChunkedShortlistMetrics, ChunkedShortlistResult,
                                ChunkedShortlistRunner)
from .graph_call import CapturedLayerCall, CapturedModelCall
from .multihead import CausalASPAMultiheadAttention
from .sparse_attn import (aspa_sparse_attention, build_packed_shortlist_candidates, build_shortlist_candidates,
                          get_last_backend, get_last_backend_info)
from .sparse_ctl import SparseHeadController
from .transformer_block import CausalASPATransformerBlock

__all__ = ["CapturedLayerCall", "CapturedModelCall", "AdaptiveSparseAttentionBlock", "AdaptiveSparseAttention", "AdaptiveSparseProtoAttention",
           "aspa_sparse_attention", "build_shortlist_candidates", "build_packed_shortlist_candidates",
           "CausalASPAMultiheadAttention", "CausalASPATransformerBlock", "SparseHeadController", "MLP", "ModelConfig",
           "get_last_backend", "get_last_backend_info", "ChunkedShortlistConfig", "ChunkedShortlistMetrics",
           "ChunkedShortlistResult", "ChunkedShortlistRunner", "__version__"]
__version__ = "0.1.0"
