#!/usr/bin/env bash
# Builds every native part in-tree (CUDA kernels for sm_100a, the placement library, the proxy) and, with --wheel,
# a wheel that carries them.  Run from anywhere; needs nvcc, g++ and python with torch.
set -euo pipefail
root="$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)"
cd "$root"
py="${PYTHON:-python3}"
"$py" -c "import __graft_entry__ as g; g.build()"
if [[ "${1:-}" == "--wheel" ]]; then
    "$py" -m pip wheel --no-deps --no-build-isolation -w "$root/dist" "$root"
    ls -l "$root/dist"
fi
