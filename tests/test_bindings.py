"""Every exported launcher of the native library must have its ctypes argument types declared: an undeclared
function receives 64-bit pointers truncated to C ints."""

import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# called only through their own ctypes declarations (tests, tuning aids)
SELF_DECLARED = {"kf_sumsq_noalloc", "kf_attn_fwd_occupancy"}


def test_all_exported_launchers_are_declared():
    exported = set()
    for path in glob.glob(os.path.join(ROOT, "csrc", "*.cu")):
        src = open(path).read()
        exported.update(re.findall(r'^(?:extern "C" )?(?:int|void\*?|void) (kf_[a-z0-9_]+)\(', src, re.M))
    declared = set(re.findall(r'"(kf_[a-z0-9_]+)":', open(os.path.join(ROOT, "kempnerforge_b200", "ops", "cuda.py")).read()))
    assert exported, "no exported launchers found"
    assert exported - declared - SELF_DECLARED == set()
