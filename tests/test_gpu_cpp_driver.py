"""The stand-alone C++ driver (csrc/flexattn_bench.cpp) must build, link against libflexattn.so without torch
or Python in the process, run the reference driver's shape (GL_main.cpp:13-16: B=1, H=4, L=2048, D=128) and exit 0."""
import json
import os
import subprocess

import pytest

EXE = os.path.join(os.path.dirname(__file__), "..", "flex_attention_tpu_b200", "flexattn_bench")


def test_driver_is_built():
    if not os.path.exists(EXE):  # a fresh checkout: build the library and the driver in-tree first
        subprocess.run(["python", os.path.join(os.path.dirname(EXE), "build.py")], check=True, timeout=1800)
    assert os.path.exists(EXE) and os.access(EXE, os.X_OK), "run python flex_attention_tpu_b200/build.py"


@pytest.mark.gpu
@pytest.mark.parametrize("extra", [[], ["--causal", "1", "--bwd", "1", "--seq", "1000"]])
def test_driver_runs(extra):
    r = subprocess.run([EXE, "--iters", "3", "--warmup", "1", *extra], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["driver"] == "flexattn_bench" and line["fwd_ms"] > 0
    assert 0.0 <= line["o0"] <= 1.0
    if extra:
        assert line["bwd_ms"] > 0
