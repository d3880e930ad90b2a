"""The drop-in boundary: the reference's own call sites compile against include/blocksparse.h,
include/fusion_blocksparse.h and include/openai_blocksparse.h, and a driver shaped like the
reference's *_fusion_test.cu programs gives the all-ones known answer on the GPU."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the reference tree: SFB_REFERENCE_DIR, else a directory `reference` beside this repository (tests skip when it is absent)
REF = os.environ.get("SFB_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
DRIVER = os.path.join(ROOT, "tests", "dropin", "driver")


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


@pytest.mark.parametrize("prog", ["no_fusion_test", "stride_fusion_test", "local_fusion_test", "big_bird_fusion_test",
                                  "fixed_fusion_test", "use_blocksparse"])
def test_reference_programs_compile_against_our_headers(tmp_path, prog):
    """The reference's test programs, unmodified, against our headers.  A quoted #include looks in the
    directory of the including file first, so the program is reached through a symbolic link in an empty
    directory (with links to the reference's validate.h / common.h, which are not ours to replace); its
    "blocksparse.h" / "fusion_blocksparse.h" then resolve to include/.  Compile only: never run."""
    if not os.path.exists(os.path.join(REF, prog + ".cu")):
        pytest.skip("reference tree not present on this machine")
    for name in (prog + ".cu", "validate.h", "common.h"):
        os.symlink(os.path.join(REF, name), tmp_path / name)
    src = str(tmp_path / (prog + ".cu"))
    out = tmp_path / (prog + ".o")
    r = subprocess.run([_nvcc(), "-std=c++14", "-arch=sm_100a", "-w", "-I", os.path.join(ROOT, "include"),
                        "-c", src, "-o", str(out)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    # every block-sparse operator the program calls resolves to our C ABI
    syms = subprocess.run(["nm", "-u", str(out)], capture_output=True, text=True).stdout
    assert "sfb_" in syms


def test_dropin_driver_builds():
    import __graft_entry__ as ge
    ge.build_dropin_driver()
    assert os.path.exists(DRIVER)


@pytest.mark.gpu
def test_dropin_driver_known_answer_on_gpu():
    if not os.path.exists(DRIVER):
        import __graft_entry__ as ge
        ge.build_dropin_driver()
    r = subprocess.run([DRIVER], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr
