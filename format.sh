#!/usr/bin/env bash
# Formats and lints the Python sources with the settings of pyproject.toml (yapf + ruff) and, when clang-format is
# installed, the C++/CUDA sources. `bash format.sh --check` only reports.
set -eo pipefail
cd "$(dirname "${BASH_SOURCE[0]}")"
check=0
[ "${1:-}" = "--check" ] && check=1
py_targets=(deepep_efa_b200 tests baseline bench.py bench_moe.py bench_gemm.py bench_kernels.py bench_normal_sweep.py __graft_entry__.py setup.py)
if command -v ruff >/dev/null; then
    if [ $check -eq 1 ]; then ruff check "${py_targets[@]}"; else ruff check --fix "${py_targets[@]}"; fi
else
    echo "ruff not installed: skipping lint" >&2
fi
if command -v yapf >/dev/null; then
    if [ $check -eq 1 ]; then yapf --diff --recursive "${py_targets[@]}"; else yapf --in-place --recursive "${py_targets[@]}"; fi
else
    echo "yapf not installed: skipping Python formatting" >&2
fi
if command -v clang-format >/dev/null; then
    files=$(find deepep_efa_b200/csrc -name '*.cu' -o -name '*.cuh' -o -name '*.h' -o -name '*.hpp' -o -name '*.cpp')
    if [ $check -eq 1 ]; then clang-format --dry-run -Werror $files; else clang-format -i $files; fi
fi
