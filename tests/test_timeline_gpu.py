"""The device timeline (kernels/timeline.py): a build of the kernels that stamps, per launch,
when its first block started and when its wait on the previous kernel returned."""
import json
import os
import subprocess
import sys

import pytest

from tests.gpu_helpers import model_dir

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_timeline_of_a_decode_step_names_every_kernel_in_order():
    env = dict(os.environ, IMPARO_TIMELINE="1")
    r = subprocess.run([sys.executable, "-m", "imparo_b200.kernels.timeline", "-m", model_dir("A"), "--batch", "3",
                        "--prompt-len", "40", "--steps", "6", "--json"], cwd=ROOT, env=env, capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    rows = json.loads(r.stdout.strip().splitlines()[-1])
    names = [x["kernel"] for x in rows]
    assert names[0].startswith("embed_gather") and names[-1].startswith(("argmax", "sample_rows")), names
    assert any(n.startswith("gated_conv") for n in names) and any("attn" in n for n in names)
    # stamps are ordered: a kernel's wait returns after the previous kernel's, and after its own start
    at = [x["at_us"] for x in rows]
    assert all(b >= a for a, b in zip(at, at[1:])), at
    assert all(x["resident_before_us"] >= 0 for x in rows)
    assert all(x["chain_us"] is None or 0 <= x["chain_us"] < 5000 for x in rows)


def test_the_normal_build_refuses_the_timeline():
    env = {k: v for k, v in os.environ.items() if k != "IMPARO_TIMELINE"}
    r = subprocess.run([sys.executable, "-c", "from imparo_b200.kernels.timeline import Timeline; Timeline()"], cwd=ROOT,
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode != 0 and "IMPARO_TIMELINE" in r.stderr
