"""Pins the CPU oracle -- and through it this library -- to outputs of the reference project's own operator run on
the same GPU: baseline/_ref/gemm_int8_CUDA.so is the reference's unmodified csrc/kernels/{gemm.cu,bindings.cpp}
compiled for sm_100 (baseline/build_reference.sh).  It registers the same torch namespace as this library, so it runs
in a process of its own (baseline/run_reference.py) and hands its bf16 results back through a file.  Cases: the
README example (config 1), the reference's test.py case, and the nine shapes of its benchmark.py:56-62 with that
script's input recipe.  Every result must equal oracle.c_matmul bit for bit, and gi8_matmul likewise.
Skipped when the reference library has not been built."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))

CASES = [{"name": "config1", "kind": "uniform", "M": 1024, "N": 4096, "K": 4096, "alpha": 1.0, "seed": 1001},
         {"name": "testpy", "kind": "testpy", "M": 32, "N": 32, "K": 32, "alpha": 1.0, "seed": 7},
         {"name": "alpha", "kind": "uniform", "M": 257, "N": 520, "K": 1040, "alpha": -3.7, "seed": 21}]
CASES += [{"name": f"bench_{m}_{n}_{k}", "kind": "benchmark", "M": m, "N": n, "K": k, "alpha": 1.0, "seed": 31 + i}
          for i, (m, n, k) in enumerate((m, n, k) for m in (512, 1024, 2048) for (n, k) in ((4096, 4096), (14336, 4096), (4096, 14336)))]


def test_reference_operator_output_equals_oracle_and_library(oracle, tmp_path):
    import run_reference

    if not run_reference.available():
        pytest.skip("baseline/_ref/gemm_int8_CUDA.so not built (baseline/build_reference.sh)")
    cases_file, out_file = tmp_path / "cases.json", tmp_path / "ref.npz"
    cases_file.write_text(json.dumps(CASES))
    res = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "run_reference.py"), "--cases", str(cases_file),
                          "--out", str(out_file)], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    ref = np.load(out_file)
    import gemm_int8_b200 as g

    for c in CASES:
        x, y = run_reference.make_case(c["kind"], c["M"], c["N"], c["K"], c["seed"])
        want = oracle.c_matmul(x, y, c["alpha"])
        got_ref = ref[c["name"]]
        assert got_ref.shape == want.shape
        assert np.array_equal(got_ref, want), f"{c['name']}: the reference operator and the oracle differ in {(got_ref != want).sum()} values"
        ours = oracle.bf16_bits(g.matmul(x.cuda(), y.cuda(), c["alpha"]))
        assert np.array_equal(ours, got_ref), c["name"]
    assert g.device_status() == 0
