"""The timeline build of the kernel library: every kernel of a replayed decode step leaves
one mark (when its first block was resident, when its predecessors had finished)."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT, require_gpu

pytestmark = pytest.mark.gpu

SCRIPT = r"""
import sys
sys.path.insert(0, sys.argv[1])
import torch
import hilbert_pruned_8b_b200 as hb
from hilbert_pruned_8b_b200.engine.step import Engine
from hilbert_pruned_8b_b200.engine.batch import StepEntry
eng = Engine.from_folder(sys.argv[2], "bfloat16", max_tokens=256)
ops = eng.ctx.ops
seqs = [eng.open_sequence() for _ in range(2)]
eng.step([StepEntry(s, [1, 2, 3], []) for s in seqs])
ops.call_log = []
eng.step([StepEntry(s, [4], [0]) for s in seqs])          # eager: its calls name the kernels
calls = [c for c in ops.call_log if c not in ("hb_device_info", "hb_timeline_set")]
ops.call_log = None
kernels = sum(2 if c == "hb_attention_decode" else 1 for c in calls)
for t in range(3):
    eng.step([StepEntry(s, [5 + t], [0]) for s in seqs])
ops.timeline_begin(4096)
steps = 4
for t in range(steps):
    eng.step([StepEntry(s, [9 + t], [0]) for s in seqs])
marks = ops.timeline_end()
assert len(marks) == kernels * steps, (len(marks), kernels, steps)
assert all(a <= b for a, b in marks), "a kernel found its predecessors finished before it was resident"
assert all(marks[i][1] <= marks[i + 1][1] for i in range(len(marks) - 1))
span_us = (marks[-1][1] - marks[0][1]) / 1e3
assert 0 < span_us < 1e6, span_us
print("ok", kernels, len(marks), round(span_us, 1))
"""


def test_every_kernel_of_a_replayed_step_leaves_a_mark(model_folders, tmp_path):
    require_gpu()
    env = dict(os.environ, HILBERT_B200_TIMELINE="1")
    script = tmp_path / "timeline_case.py"
    script.write_text(SCRIPT)
    res = subprocess.run([sys.executable, str(script), ROOT, model_folders["strong_d"]], env=env, capture_output=True,
                         text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.strip().startswith("ok")
