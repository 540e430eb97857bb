#!/usr/bin/env bash
# Compile the sm_100a extension in-tree and build a wheel into dist/.
set -euo pipefail
cd "$(dirname "$0")"
python setup.py build_ext --inplace
python -m pip wheel --no-deps --no-build-isolation -w dist .
