"""Link-level drop-in check: the reference's own benchmark driver (SSpMM/sspmm_test.cpp, compiled
unmodified by `make -C oracle dropin` and linked against libsspmm_b200.so) reads a CVSE .smtx file
written by the GPU SVC, calls spmm::SSpMM / spmm::SpMM from our library and verifies the result
against its own host loop (SSpMM/sspmm_test.cpp:75-95, 230-253)."""
import os
import subprocess

import pytest

from sspmm_b200 import synthetic

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVER = os.path.join(ROOT, "oracle", "_ref", "sspmm_test_dropin")


@pytest.mark.skipif(not os.path.exists(DRIVER), reason="reference driver not built (make -C oracle dropin)")
@pytest.mark.parametrize("V,kernel,mixed", [(8, 1, 0), (16, 1, 1), (16, 0, 0), (8, 1, 1)])
def test_reference_driver_runs_on_our_library(lib, tmp_path, V, kernel, mixed):
    from sspmm_b200 import sparse_matrix_format as smf
    a, _ = synthetic.config1()
    c = smf.CVSE(a.M, a.K, a.nnz, a.row_lists(), V)
    # the driver looks for ../benchmark/dlmc-v{8,16}/<name> relative to its working directory (:313-334)
    bench = tmp_path / "benchmark" / f"dlmc-v{V}"
    bench.mkdir(parents=True)
    c.CVSE_out(str(bench / "config1.smtx"))
    run = tmp_path / "run"
    run.mkdir()
    (run / "paths.txt").write_text("config1.smtx\n")
    #            paths      N      V       kernel       sort verify mixed      record reorder arch
    args = [DRIVER, "paths.txt", "256", str(V), str(kernel), "1", "1", str(mixed), "0", "0", "b200"]
    r = subprocess.run(args, cwd=run, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Results verified: they agree." in r.stdout, r.stdout[-2000:]
    assert "matrix num:1" in r.stdout
