#!/usr/bin/env bash
# Release gate: no machine-specific paths in the tree, every shell script parses, every Python file compiles, the
# CUDA sources cross-compile for sm_100a (when nvcc is present), and the CPU test-suite passes.
set -euo pipefail
cd "$(dirname "${BASH_SOURCE[0]}")"
py="${PYTHON:-python}"

if git ls-files -z | xargs -0 grep -InE '/home/[a-z]+/|/mnt/[a-z]+/|(^|[^0-9])(10|172|192)\.[0-9]+\.[0-9]+\.[0-9]+' -- \
     ':!validate_release.sh' 2>/dev/null | grep -v '127\.0\.0\.1'; then
  echo "validate_release: machine-specific path or address found" >&2
  exit 1
fi
echo "path scan: clean"

git ls-files '*.sh' | while read -r f; do bash -n "$f"; done
echo "shell syntax: ok"

"$py" - <<'PY'
import pathlib, subprocess, sys
files = subprocess.run(["git", "ls-files", "*.py"], capture_output=True, text=True).stdout.split()
bad = []
for f in files:
    try:
        compile(pathlib.Path(f).read_bytes(), f, "exec")
    except Exception as exc:
        bad.append((f, exc))
print(f"python syntax: {len(files) - len(bad)} ok, {len(bad)} failed")
for f, exc in bad:
    print(f"  {f}: {exc}")
sys.exit(1 if bad else 0)
PY

if command -v nvcc >/dev/null 2>&1; then
  for f in terra_b200/csrc/*.cu; do
    nvcc -gencode arch=compute_100a,code=sm_100a -std=c++17 -O1 -c "$f" -o /dev/null
  done
  echo "sm_100a cross-compile: ok"
fi

"$py" -m pytest -q tests -m "not gpu" "$@"
