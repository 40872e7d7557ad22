"""B200-native SparseConv2D for SV-TAD: the hot path of pcr-upm/eccv26_tad behind its own call surface."""
from .sparse_conv_layer import SparseConv2d, SparseConv2dFunction, remap_legacy_sparse_conv_weights  # noqa: F401
from .neighbor_table import (  # noqa: F401
    build_neighbor_table,
    get_initial_neighbor_indices,
    num_keep_tokens,
    select_and_update,
    select_topk,
    update_neighbor_indices,
)
from .backbone import SparseAdapterViT  # noqa: F401,E402
