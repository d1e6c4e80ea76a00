"""The reference's own test scripts, unmodified, against this library: ``import deep_ep`` resolves to the drop-in module
in ``deepep_efa_b200/compat``. The scripts are the copies that ``baseline/build_reference.py`` places beside the
reference build (``baseline/_ref/ref_tests``); without them, or with fewer than two GPUs, the tests are skipped."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
REF_TESTS = ROOT / "baseline" / "_ref" / "ref_tests"


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("script,extra", [
    ("test_intranode.py", []),                          # 4096 tokens, hidden 7168, 256 experts, top-8: checks + its tuning sweep
    ("test_low_latency.py", ["--num-experts", "256"]),  # 128 tokens, hidden 7168, top-8: checks, hooks, zero-copy, its benchmark
])
def test_reference_script_passes_against_this_library(script, extra):
    if not (REF_TESTS / script).is_file():
        pytest.skip("reference test scripts not present (run baseline/build_reference.py)")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    # two ranks by default (enough to cross NVLink and quick); DEEPEP_TEST_REF_WORLD=4|8 runs the scripts' full size
    world = min(int(os.environ.get("DEEPEP_TEST_REF_WORLD", "2")), torch.cuda.device_count())
    env = os.environ.copy()
    env["PYTHONPATH"] = os.pathsep.join([str(ROOT / "deepep_efa_b200" / "compat"), str(ROOT), env.get("PYTHONPATH", "")])
    env.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE="1", RANK="0", NCCL_NVLS_ENABLE="0")
    proc = subprocess.run([sys.executable, str(REF_TESTS / script), "--num-processes", str(world)] + extra, env=env, cwd=str(REF_TESTS),
                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=900)
    tail = "\n".join(proc.stdout.splitlines()[-40:])
    assert proc.returncode == 0, f"{script} failed:\n{tail}"
    assert "Traceback" not in proc.stdout, tail
