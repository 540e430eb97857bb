#!/usr/bin/env bash
# Format or check the sources.  Python: ruff (lint + import order) and yapf, settings in pyproject.toml.  C++ / CUDA:
# clang-format with .clang-format.  A tool that is not installed is reported and skipped.
#   ./format.sh            rewrite files that were changed with respect to origin/main (or all files without git)
#   ./format.sh --all      every tracked source file
#   ./format.sh --check    change nothing; exit 1 if ruff reports a finding; files that yapf / clang-format would rewrite are listed
#   ./format.sh --check --strict    also exit 1 for files that yapf / clang-format would rewrite
set -uo pipefail
cd "$(dirname "$0")"

mode=changed
check=0
strict=0
for arg in "$@"; do
    case "$arg" in
        --all) mode=all ;;
        --check) check=1 ;;
        --strict) strict=1 ;;
        -h|--help) sed -n 2,8p "$0"; exit 0 ;;
        *) echo "unknown argument: $arg" >&2; exit 2 ;;
    esac
done

list_files() {   # $1: extended regular expression on the path
    if [ "$mode" = all ] || ! git rev-parse --git-dir > /dev/null 2>&1; then
        git ls-files 2> /dev/null | grep -E "$1" || find deepep_ascend_b200 tests -type f | grep -E "$1"
    else
        base=$(git merge-base HEAD origin/main 2> /dev/null || git rev-list --max-parents=0 HEAD | tail -1)
        { git diff --name-only --diff-filter=ACMR "$base"; git ls-files --others --exclude-standard; } | sort -u | grep -E "$1"
    fi
}

status=0
py_files=$(list_files '\.py$' | grep -v '^baseline/' || true)
cc_files=$(list_files '\.(cu|cuh|cpp|hpp|h)$' || true)

if [ -n "$py_files" ]; then
    if command -v ruff > /dev/null; then
        if [ $check = 1 ]; then ruff check $py_files || status=1; else ruff check --fix $py_files || status=1; fi
    else
        echo "ruff is not installed: Python lint skipped"
    fi
    if command -v yapf > /dev/null; then
        if [ $check = 1 ]; then yapf --diff $py_files > /dev/null || { echo "yapf would reformat Python files"; [ $strict = 1 ] && status=1; }
        else yapf --in-place $py_files; fi
    else
        echo "yapf is not installed: Python formatting skipped"
    fi
fi
if [ -n "$cc_files" ]; then
    if command -v clang-format > /dev/null; then
        if [ $check = 1 ]; then clang-format --dry-run --Werror $cc_files > /dev/null 2>&1 || { echo "clang-format would rewrite C++ / CUDA files"; [ $strict = 1 ] && status=1; }
        else clang-format -i $cc_files; fi
    else
        echo "clang-format is not installed: C++ / CUDA formatting skipped"
    fi
fi
exit $status
