"""The C ABI from C: tests/c_client.c is compiled against include/llmtie_b200.h
with plain gcc, linked to the library and to the oracle (as its checker), and
run. No Python or torch is on that program's path."""
import os
import shutil
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_a_plain_c_caller_prefills_and_decodes(gpu, tmp_path):
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler on this box")
    from oracle import oracle as O

    O.lib()   # builds oracle/liboracle.so if it is not there yet
    libdir = os.path.join(ROOT, "ttsxabe_b200")
    oradir = os.path.join(ROOT, "oracle")
    exe = str(tmp_path / "c_client")
    build = subprocess.run(
        [gcc, "-O2", "-std=gnu11", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", oradir,
         os.path.join(ROOT, "tests", "c_client.c"), "-o", exe, "-L", libdir, "-lllmtie_b200",
         "-L", oradir, "-loracle", "-lm", "-Wl,-rpath," + libdir, "-Wl,-rpath," + oradir],
        capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    sys.stdout.write(run.stdout)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "all checks passed" in run.stdout
