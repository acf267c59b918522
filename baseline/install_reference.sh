#!/usr/bin/env bash
# Install the unmodified reference (mega_up 0.3.0) into baseline/_ref (git-ignored)
# from a checkout given as $1, plus its test and benchmark runners, which the
# package does not ship: bench.py's reference arm imports the unfused torch
# baselines from them, and megaup_b200.benchmark's `reference_fused` column runs
# the reference's own kernels from the installed package on one GPU.
#
#   bash baseline/install_reference.sh /path/to/reference
set -euo pipefail
SRC="${1:?usage: install_reference.sh /path/to/reference}"
HERE="$(cd "$(dirname "$0")" && pwd)"
TMP="$(mktemp -d)"
cp -r "$SRC" "$TMP/ref"            # the build writes into the source tree
rm -rf "$HERE/_ref"
python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
    --target "$HERE/_ref" "$TMP/ref"
mkdir -p "$HERE/_ref/reference_runners"
cp "$SRC"/tests/*.py "$HERE/_ref/reference_runners/"
cp "$SRC"/benchmarks/*.py "$HERE/_ref/reference_runners/" 2>/dev/null || true
rm -rf "$TMP"
echo "installed into $HERE/_ref"
