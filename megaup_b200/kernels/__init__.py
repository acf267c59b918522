"""Host-side handles of the two sm_100a kernels in libmegaup.so."""

from .headshard_pull_gemm import CompiledHeadShardPullGemm, compile_headshard_pull_gemm
from .peer_write_gemm import PeerWriteLaunch, make_peer_write_launch, peer_n_rotation

__all__ = [
    "CompiledHeadShardPullGemm",
    "PeerWriteLaunch",
    "compile_headshard_pull_gemm",
    "make_peer_write_launch",
    "peer_n_rotation",
]
