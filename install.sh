#!/usr/bin/env bash
# Build the wheel and install it into the current environment.
set -euo pipefail
cd "$(dirname "$0")"
./build.sh
python -m pip install --no-deps --force-reinstall dist/deepep_ascend_b200-*.whl
