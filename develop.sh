#!/usr/bin/env bash
# In-place development build: compile the extension and put the repository on the path of the current environment.
set -euo pipefail
cd "$(dirname "$0")"
python setup.py build_ext --inplace
python -m pip install --no-deps --no-build-isolation -e .
