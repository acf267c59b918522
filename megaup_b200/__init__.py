"""B200-native fused GEMM + Ulysses all-to-all operators behind the ``mega_up`` API.

Two operators, forward only, BF16 in / FP32 accumulate / one rounding to BF16,
one node, ``UP`` in {2, 4, 8}:

* peer-write GEMM - ``x @ W.T + b`` whose epilogue stores every head shard
  straight into the owning rank's arena slot (replaces linear + permute +
  all_to_all);
* head-shard pull GEMM - pull warps gather every peer's head shard of each row
  while the MMA warps consume finished panels (replaces all_to_all + permute +
  linear).

The device code is hand-written sm_100a CUDA in ``libmegaup.so`` (C ABI in
``include/megaup.h``); this package is the host side.
"""

from .ops import (
    PreparedHeadShardPullGemm,
    PreparedHeadShardPullGemmSBHD,
    PreparedHeadShardPullGemmTHD,
    PreparedPeerWriteGemm,
    PreparedPeerWriteGemmSBHD,
    PreparedPeerWriteGemmTHD,
    THDLayout,
    emulated_peer_write,
    emulated_pull,
    headshard_pull_gemm_bshd,
    headshard_pull_gemm_sbhd,
    headshard_pull_gemm_thd,
    peer_write_gemm_bshd,
    peer_write_gemm_sbhd,
    peer_write_gemm_thd,
    prepare_headshard_pull_gemm_bshd,
    prepare_headshard_pull_gemm_sbhd,
    prepare_headshard_pull_gemm_thd,
    prepare_peer_write_gemm_bshd,
    prepare_peer_write_gemm_sbhd,
    prepare_peer_write_gemm_thd,
    prepare_thd_layout,
)
from .runtime import (
    DEFAULT_MAX_ROWS,
    SUPPORTED_UP_DEGREES,
    MegaUPRuntime,
    initialize_emulated_group,
    initialize_runtime,
    supports_shape,
    unsupported_shape_reason,
)

__version__ = "0.1.0"

__all__ = [
    "DEFAULT_MAX_ROWS",
    "SUPPORTED_UP_DEGREES",
    "MegaUPRuntime",
    "PreparedHeadShardPullGemm",
    "PreparedHeadShardPullGemmSBHD",
    "PreparedHeadShardPullGemmTHD",
    "PreparedPeerWriteGemm",
    "PreparedPeerWriteGemmSBHD",
    "PreparedPeerWriteGemmTHD",
    "THDLayout",
    "emulated_peer_write",
    "emulated_pull",
    "headshard_pull_gemm_bshd",
    "headshard_pull_gemm_sbhd",
    "headshard_pull_gemm_thd",
    "initialize_emulated_group",
    "initialize_runtime",
    "peer_write_gemm_bshd",
    "peer_write_gemm_sbhd",
    "peer_write_gemm_thd",
    "prepare_headshard_pull_gemm_bshd",
    "prepare_headshard_pull_gemm_sbhd",
    "prepare_headshard_pull_gemm_thd",
    "prepare_peer_write_gemm_bshd",
    "prepare_peer_write_gemm_sbhd",
    "prepare_peer_write_gemm_thd",
    "prepare_thd_layout",
    "supports_shape",
    "unsupported_shape_reason",
]
