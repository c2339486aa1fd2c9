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
