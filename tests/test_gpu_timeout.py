"""A device-side wait that runs out: the kernel must return by itself, report
``B200_SDPA_ERR_TIMEOUT`` through the status word and leave the context usable.

This is the library's counterpart of upstream's collective watchdog
(``torch_neuronx/csrc/distributed/NeuronWatchdog.h:16-31``: a stuck device operation is
noticed and reported instead of hanging the process).  Nothing is injected and nothing
faults: a child process sets the wait limit to a few dozen cycles (``B200_SDPA_WAIT_LIMIT``,
read once per process), so the first barrier wait of a one-CTA prefill that is not satisfied at
once gives up; every role then drains, the CTA waits for the copies and MMAs it already issued,
frees its tensor memory and exits.  A second child runs the same call with the default limit
and checks it against the oracle.
"""

import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import json, sys, torch
sys.path.insert(0, {root!r})
import torch_neuronx_b200 as T
from oracle import sdpa_oracle as O

dev = torch.device("cuda", 0)
g = torch.Generator().manual_seed(7)
q = torch.randn(1, 1, 128, 128, generator=g).to(torch.bfloat16)
k = torch.randn(1, 1, 256, 128, generator=g).to(torch.bfloat16)
v = torch.randn(1, 1, 256, 128, generator=g).to(torch.bfloat16)
res = {{}}
T.reset_launch_counts()
out, lse = T.sdpa_forward(q.to(dev), k.to(dev), v.to(dev), scale=0.1)
torch.cuda.synchronize()
res["grid"] = list(T.ops.last_plan["grid"])
res["prefill_launches"] = T.launch_counts()["prefill"]
try:
    T.check_device_status()
    res["status"] = "ok"
except RuntimeError as e:
    res["status"] = str(e)
ref_o, ref_l = O.sdpa_forward(q, k, v, scale=0.1, compute_dtype=torch.float32)
res["max_abs"] = float((out.cpu().float() - ref_o).abs().nan_to_num(1e9).max())
# the context must still work: a torch kernel and a kernel of this library without barrier waits
x = torch.arange(1000, device=dev).sum().item()
res["torch_ok"] = x == 499500
o2, _ = T.sdpa_forward(q.float().to(dev), k.float().to(dev), v.float().to(dev), scale=0.1)
torch.cuda.synchronize()
res["generic_max_abs"] = float((o2.cpu() - O.sdpa_forward(q.float(), k.float(), v.float(), scale=0.1)[0]).abs().max())
print("RESULT " + json.dumps(res))
"""


def _run_child(extra_env):
    env = dict(os.environ)
    env.pop("B200_SDPA_WAIT_LIMIT", None)
    env.update(extra_env)
    proc = subprocess.run([sys.executable, "-c", CHILD.format(root=ROOT)], env=env, capture_output=True, text=True,
                          timeout=300)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    line = [ln for ln in proc.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


@pytest.mark.parametrize("form", ["per_cta", "persistent"])
def test_a_wait_that_runs_out_is_reported_and_the_context_survives(form):
    # both forms of the prefill kernel (one item per CTA; persistent CTAs) have the same give-up path
    res = _run_child({"B200_SDPA_WAIT_LIMIT": "64", "B200_SDPA_PREFILL": form})
    assert res["grid"][0] == 1 and res["prefill_launches"] == 1          # one CTA of the tensor-core kernel
    assert "device status 10" in res["status"] and "gave up" in res["status"], res
    assert res["torch_ok"] and res["generic_max_abs"] <= 1e-5, res       # the context kept working


@pytest.mark.parametrize("form", ["per_cta", "persistent"])
def test_the_same_call_with_the_default_limit_is_correct(form):
    res = _run_child({"B200_SDPA_PREFILL": form})
    assert res["status"] == "ok" and res["prefill_launches"] == 1, res
    assert res["max_abs"] <= 2e-2, res
