"""Every sub-command of ``python -m crane_b200.profiling`` runs at a small size
and prints one JSON record: the commands that the kernel summaries under
profiles/ were taken with stay runnable."""
import json

import pytest

pytestmark = pytest.mark.gpu

CASES = [
    ["gemm", "--m", "8", "--n", "512", "--k", "256"],
    ["gemm", "--m", "256", "--n", "512", "--k", "256"],
    ["gemm", "--m", "256", "--n", "512", "--k", "256", "--silu-mul"],
    ["gemm", "--m", "512", "--n", "512", "--k", "256", "--pair"],
    ["decode-attention", "--batch", "2", "--context", "300"],
    ["decode-attention", "--batch", "8", "--context", "1024"],
    ["decode-attention", "--batch", "3", "--context", "200", "--head-dim", "64", "--q-heads", "6", "--kv-heads", "2"],
    ["prefill-attention", "--tokens", "300"],
    ["prefill-attention", "--tokens", "300", "--kernel", "mma"],
    ["rmsnorm", "--rows", "64", "--hidden", "768"],
]


@pytest.mark.parametrize("argv", CASES, ids=lambda a: " ".join(a))
def test_profiling_command_runs(argv, capsys):
    from crane_b200 import profiling
    assert profiling.main(["--warmup", "1", "--reps", "2"] + argv) == 0
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rec["us"] > 0 and rec["kernel"]


def test_tall_tile_commands_run(capsys):
    from crane_b200 import profiling
    for argv in (["gemm", "--m", "512", "--n", "384", "--k", "256", "--bn", "192", "--tall"],
                 ["gemm", "--m", "1024", "--n", "512", "--k", "256", "--bn", "256", "--pair", "--tall"]):
        assert profiling.main(["--warmup", "1", "--reps", "2"] + argv) == 0
        rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert rec["us"] > 0 and rec["tile_rows"] in (256, 512)


def test_hardware_measurements_run(capsys):
    """One thread's issue rate of tcgen05.mma and the cost of a barrier across
    the SMs: every product completes, no wait runs out, and the figures are of
    the order the kernels' designs assume."""
    from crane_b200 import profiling
    assert profiling.main(["hardware"]) == 0
    recs = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    mma = [r for r in recs if "cycles_per_product_issue_loop" in r]
    bar = [r for r in recs if "cycles_per_barrier" in r]
    assert len(mma) == 3 and len(bar) == 3
    for r in mma:
        assert r["completed"] and r["tensor_core_cycles_per_product"] * 0.9 <= r["cycles_per_product_until_complete"] < 400
    for r in bar:
        assert not r["wait_ran_out"] and 200 < r["cycles_per_barrier"] < 20000
