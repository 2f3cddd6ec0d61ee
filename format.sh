#!/usr/bin/env bash
# Format check of the repository (the counterpart of the reference's format.sh and its GitHub workflow
# .github/workflows/format.yml): Python through ruff when it is installed, otherwise a byte-compile of every file;
# C++ / CUDA through clang-format --dry-run when it is installed. Exits non-zero on a finding.
set -u
cd "$(dirname "$0")"
status=0
if command -v ruff > /dev/null 2>&1; then
    ruff check deepep_b200 tests bench.py __graft_entry__.py setup.py || status=1
else
    python -m compileall -q deepep_b200 tests bench.py __graft_entry__.py setup.py > /dev/null || status=1
fi
if command -v clang-format > /dev/null 2>&1; then
    find deepep_b200/csrc \( -name '*.cu' -o -name '*.cuh' -o -name '*.hpp' -o -name '*.cpp' -o -name '*.h' \) -print0 |
        xargs -0 clang-format --dry-run --Werror || status=1
fi
exit $status
