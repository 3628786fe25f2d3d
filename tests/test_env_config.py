"""The two environment variables that set the default convolution algorithms
(warpconvnet/constants.py:95-117 of the reference): value, list syntax, rejection of unknown
values, and that a module built without an explicit algorithm picks them up."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROBE = """
import json
from warpconvnet_b200 import constants
from warpconvnet_b200.nn.modules.sparse_conv import SparseConv3d
m = SparseConv3d(4, 4, 3)
print(json.dumps({"fwd": constants.WARPCONVNET_FWD_ALGO_MODE, "bwd": constants.WARPCONVNET_BWD_ALGO_MODE,
                  "mod_fwd": getattr(m.fwd_algo, "value", m.fwd_algo), "mod_bwd": getattr(m.bwd_algo, "value", m.bwd_algo)}))
"""


def run(env):
    e = {k: v for k, v in os.environ.items() if not k.startswith("WARPCONVNET_")}
    e.update(env)
    e["PYTHONPATH"] = ROOT + os.pathsep + e.get("PYTHONPATH", "")
    return subprocess.run([sys.executable, "-c", PROBE], env=e, capture_output=True, text=True, timeout=300)


def test_defaults_are_auto():
    import json
    r = run({})
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out == {"fwd": "auto", "bwd": "auto", "mod_fwd": "auto", "mod_bwd": "auto"}


def test_values_and_lists_are_parsed():
    import json
    r = run({"WARPCONVNET_FWD_ALGO_MODE": "Implicit_GEMM", "WARPCONVNET_BWD_ALGO_MODE": "[explicit_gemm, 'cutlass_implicit_gemm']"})
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["fwd"] == "implicit_gemm" and out["mod_fwd"] == "implicit_gemm"
    assert out["bwd"] == ["explicit_gemm", "cutlass_implicit_gemm"] and out["mod_bwd"] == ["explicit_gemm", "cutlass_implicit_gemm"]


def test_unknown_values_are_rejected():
    r = run({"WARPCONVNET_FWD_ALGO_MODE": "winograd"})
    assert r.returncode != 0 and "WARPCONVNET_FWD_ALGO_MODE" in r.stderr
    r = run({"WARPCONVNET_BWD_ALGO_MODE": "[implicit_gemm,fft]"})
    assert r.returncode != 0 and "WARPCONVNET_BWD_ALGO_MODE" in r.stderr
