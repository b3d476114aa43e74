#!/usr/bin/env bash
# Installs the unmodified reference package into baseline/_ref (git-ignored) for the head-to-head bench arm.
# 1) the regular offline pip install; 2) if the build backend is not available offline (the reference builds
# with hatchling), fall back to copying the pure-Python package directory verbatim — a hatchling wheel of a
# pure-Python project contains exactly this directory.
set -u
here="$(cd "$(dirname "$0")" && pwd)"
ref="${1:-${KF_REFERENCE_ROOT:-$here/../../reference}}"   # the reference checkout: argument, KF_REFERENCE_ROOT, or beside this repository
wheels="${KF_WHEELHOUSE:-/opt/wheelhouse}"
target="$here/_ref"
mkdir -p "$target"
if python -m pip install --no-index --no-build-isolation --find-links "$wheels" --no-deps --target "$target" "$ref" \
     > "$here/_ref_pip.log" 2>&1; then
  echo "pip install ok" | tee "$target/INSTALL_METHOD"
else
  echo "pip install failed (see baseline/_ref_pip.log); copying the pure-Python package verbatim" >&2
  rm -rf "$target/kempnerforge"
  cp -r "$ref/kempnerforge" "$target/kempnerforge"
  echo "verbatim copy of $ref/kempnerforge (pip: $(tail -1 "$here/_ref_pip.log"))" > "$target/INSTALL_METHOD"
fi
python - <<PY
import sys; sys.path.insert(0, "$target")
import kempnerforge; print("reference importable from", kempnerforge.__file__)
PY
