"""The bounds-checked build of the library (-DDECODE_ATTN_BOUNDS_CHECK, libdecode_attn_checked.so): out-of-bounds
block indices and foreign block pointers are recorded (DX_ERR_BOUNDS) and redirected instead of followed, results of
clean steps are unchanged.  The cases run in a process of their own (tests/bounds_check_cases.py), because a process
loads one build of the library."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CHECKED = ROOT / "tensorrt-llm_b200" / "libdecode_attn_checked.so"


def test_regular_build_has_no_checks(pkg):
    assert pkg.load_library().dx_build_has_bounds_check() == 0


@pytest.mark.gpu
def test_checked_build_reports_and_redirects(pkg):
    assert CHECKED.exists(), "build it with: python tensorrt-llm_b200/build.py --checked (build() does)"
    env = dict(os.environ, DX_DECODE_ATTN_LIB=str(CHECKED))
    r = subprocess.run([sys.executable, str(ROOT / "tests" / "bounds_check_cases.py")], env=env, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    res = json.loads(r.stdout.strip().splitlines()[-1])
    assert res["has_checks"] == 1
    bounds = pkg.plugin.DX_ERR_BOUNDS
    for name, c in res.items():
        if name == "has_checks":
            continue
        assert c["clean_parity"], name
        # (the feature-complete kernels never walk more slots than the table has: nothing to report there)
        assert c["index_beyond_row"] == bounds or (name.startswith("general") and c["index_beyond_row"] == 0), (name, c)
        assert c["index_beyond_row_cleared"] == 0, (name, c)
        assert c["inside_pool"] == 0, (name, c)
        assert c["pointer_outside_pool"] == bounds, (name, c)
        assert c["foreign_untouched"], name
        assert c["clean_parity_after"], name


@pytest.mark.gpu
def test_checked_build_passes_the_feature_and_multi_token_parity_tests(pkg):
    """The checks sit in every block-table look-up, including the per-row look-ups of the feature forms: the parity
    tests of beams / windows / ALiBi / draft tokens must come out the same on the checked build."""
    assert CHECKED.exists()
    env = dict(os.environ, DX_DECODE_ATTN_LIB=str(CHECKED))
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu",
                        str(ROOT / "tests" / "test_generation_features_gpu.py"), "-k", "against_oracle",
                        str(ROOT / "tests" / "test_multi_token_gpu.py")],
                       env=env, capture_output=True, text=True, timeout=900, cwd=str(ROOT))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout and "failed" not in r.stdout
