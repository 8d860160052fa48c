#!/usr/bin/env bash
# Checks to run before a commit: deploy/pre_commit.sh [--fast] [--fix]
#
#   1. no build product or ignored scratch file is staged (*.so, *.o, build/, anything .gitignore lists)
#   2. every shell script parses (bash -n), every Python file compiles
#   3. formatting and import order with ruff when it is installed (--fix rewrites instead of complaining)
#   4. the CUDA sources compile for sm_100a (skipped with --fast, or when nvcc is absent)
#   5. the CPU test suite (a quick subset with --fast)
source "$(dirname -- "${BASH_SOURCE[0]}")/lib.sh"
fast=0 fix=0
for a in "$@"; do case "$a" in --fast) fast=1 ;; --fix) fix=1 ;; *) fail "unknown option $a" ;; esac; done
cd "${REPO_DIR}"

say "1/5 staged files"
if git rev-parse --git-dir >/dev/null 2>&1; then
    staged="$(git diff --cached --name-only)"
    bad="$(grep -E '(\.so|\.o|\.a)$|(^|/)build/' <<<"${staged}" || true)"
    # a file that .gitignore lists can still be staged with `git add -f`: refuse those as well
    ignored="$([[ -z "${staged}" ]] || git check-ignore --no-index ${staged} 2>/dev/null || true)"
    [[ -z "${bad}${ignored}" ]] || fail "build products or ignored scratch files are staged:"$'\n'"${bad}${ignored}"
fi

say "2/5 syntax"
while IFS= read -r f; do bash -n "$f" || fail "shell syntax: $f"; done < <(git ls-files '*.sh' 2>/dev/null || find deploy -name '*.sh')
python3 -m compileall -q astrai_b200 tests bench.py __graft_entry__.py >/dev/null || fail "a Python file does not compile"

say "3/5 format"
if command -v ruff >/dev/null 2>&1; then
    if (( fix )); then ruff format astrai_b200 tests bench.py && ruff check --select I --fix astrai_b200 tests bench.py
    else ruff format --check astrai_b200 tests bench.py && ruff check --select I astrai_b200 tests bench.py; fi
else
    say "ruff is not installed: skipped"
fi

say "4/5 CUDA build"
if (( ! fast )) && command -v nvcc >/dev/null 2>&1; then python3 -m astrai_b200.ops.build >/dev/null; else say "skipped"; fi

say "5/5 tests"
if (( fast )); then python3 -m pytest tests/test_core.py tests/test_data.py tests/test_models.py -x -q -m "not gpu"
else python3 -m pytest tests -x -q -m "not gpu"; fi
say "all checks passed"
