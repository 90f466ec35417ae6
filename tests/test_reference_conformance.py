"""The reference's own CPU tests of the typed front end, run against this package (``tilefish`` aliased to ``tilefish_b200``).

Only when the reference checkout is present (it is not on a GPU box; the tests then skip). Each file runs in a child pytest
with the alias plugin. Tests that cannot pass here are listed below WITH the reason; the check is two-sided: a test that
fails without being listed fails this module, and so does a listed test that passes (the list cannot go stale).

Files of the reference's suite that are left out altogether, and why:
  test_alignment.py  ``tilefish.aot`` compile specs for Triton (pointer-alignment specialisation of generated Triton kernels)
"""

import os
import subprocess
import sys
import xml.etree.ElementTree as ET

import pytest

REF_TESTS = "/root/reference/python/tests"
HERE = os.path.dirname(os.path.abspath(__file__))

TRITON = "names a Triton type or lowers through Triton: there is no Triton in this backend"

# file -> (tests that must pass at least, {test id (prefix) -> why it cannot pass here})
EXPECTED = {
    "test_types.py": (15, {}),
    "test_dims.py": (54, {}),
    "test_graphs.py": (5, {}),
    "test_dtypes.py": (128, {
        "test_triton_pointer_names": TRITON,
        "test_triton_scalar_names": TRITON,
    }),
    "test_copy.py": (31, {
        "test_compile_specs_survive_copy_and_pickle": "tilefish.aot: compile specs of Triton kernels",
    }),
    "test_trace.py": (67, {}),
    "test_calls.py": (28, {}),
    "test_readme.py": (4, {
        "test_readme_gelu_extern_produces_a_spec": "tilefish.aot: compile specs of Triton kernels",
        "test_the_masks_section_runs_and_lowers": "the lowering guide's masked loads (DevScalar) exist for the Triton lowering only",
    }),
}


def run_file(name, tmp_path):
    xml = tmp_path / (name + ".xml")
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1", PYTHONPATH=HERE + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.run([sys.executable, "-m", "pytest", "-p", "conformance_alias", "-p", "no:cacheprovider", "-q", "--no-header", f"--junitxml={xml}", name],
                          cwd=REF_TESTS, env=env, capture_output=True, text=True, timeout=600)
    assert xml.exists(), proc.stdout[-2000:] + proc.stderr[-2000:]
    passed, failed = [], []
    for case in ET.parse(xml).getroot().iter("testcase"):
        bad = any(child.tag in ("failure", "error") for child in case)
        skipped = any(child.tag == "skipped" for child in case)
        if not skipped:
            (failed if bad else passed).append(case.get("name"))
    return passed, failed


@pytest.mark.skipif(not os.path.isdir(REF_TESTS), reason="the reference checkout is not on this machine")
@pytest.mark.parametrize("name", sorted(EXPECTED))
def test_reference_file(name, tmp_path):
    at_least, gaps = EXPECTED[name]
    passed, failed = run_file(name, tmp_path)
    unexplained = [t for t in failed if not any(t.startswith(g) for g in gaps)]
    assert not unexplained, f"{name}: fail without a listed reason: {unexplained}"
    stale = [g for g in gaps if not any(t.startswith(g) for t in failed)]
    assert not stale, f"{name}: listed as a gap but passes (or no longer exists): {stale}"
    assert len(passed) >= at_least, f"{name}: {len(passed)} passed, expected at least {at_least}"
