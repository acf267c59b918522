"""Import alias: ``import mega_up`` resolves to the B200-native implementation in
``megaup_b200``, including the submodules the reference's tests and benchmark
import (``mega_up.ops``, ``mega_up.runtime``, ``mega_up.kernels.*``)."""

import importlib
import sys

import megaup_b200
from megaup_b200 import *  # noqa: F401,F403
from megaup_b200 import __all__, __version__  # noqa: F401

for _name in ("ops", "runtime", "kernels", "kernels.peer_write_gemm", "kernels.headshard_pull_gemm"):
    sys.modules[f"{__name__}.{_name}"] = importlib.import_module(f"megaup_b200.{_name}")
ops = sys.modules[f"{__name__}.ops"]
runtime = sys.modules[f"{__name__}.runtime"]
kernels = sys.modules[f"{__name__}.kernels"]
del importlib, sys, _name
