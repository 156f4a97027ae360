"""The benchmark driver's host-side contract: configurations, the shared `config` object of both arms, clean exits
on a machine without a GPU."""

import json
import subprocess
import sys

import pytest

import bench
from torchure_b200.config import validate_config


@pytest.mark.parametrize("parallel,n", [("dp", 1), ("dp", 2), ("dp", 8), ("fsdp", 8), ("hsdp2", 8), ("tp2", 2),
                                        ("tp2sp", 2), ("tp2lp", 8), ("cp2", 2)])
def test_bench_configs_are_valid_and_keep_the_headline_shape(parallel, n):
    cfg = bench.bench_config("0.6b", n, 30, parallel=parallel)
    validate_config(cfg, n)
    assert cfg["data"]["seq_len"] == 4096 and cfg["data"]["micro_batch_size"] == 2
    mc = cfg["model"]["config"]
    assert (mc["num_layers"], mc["emb_dim"], mc["ffn_dim"], mc["vocab_size"]) == (28, 1024, 3072, 151936)
    replicas = n // (cfg["mesh"].get("tp", 1) * cfg["mesh"].get("cp", 1))
    assert cfg["data"]["global_batch_size"] == 2 * replicas      # weak scaling: 2 sequences per data-parallel rank


def test_both_arms_print_the_same_config_object():
    cfg = bench.bench_config("0.6b", 8, 30)
    a, b = bench.shared_config("0.6b", cfg, 8, 4096), bench.shared_config("0.6b", json.loads(json.dumps(cfg)), 8, 4096)
    assert a == b and a["parallelism"] == "dp8" and a["global_batch"] == 16 and a["seq_len"] == 4096
    lp = bench.bench_config("0.6b", 2, 30, parallel="tp2lp")
    lp["tp"] = {"loss_parallel": True}
    assert bench.shared_config("0.6b", lp, 2, 4096)["parallelism"] == "dp1xtp2+loss_parallel"


@pytest.mark.parametrize("impl", ["ours", "reference"])
def test_arms_exit_cleanly_without_a_gpu(impl):
    import torch

    if torch.cuda.is_available():
        pytest.skip("needs a machine without a GPU")
    out = subprocess.run([sys.executable, "bench.py", "--impl", impl, "--gpus", "1", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=120, cwd=bench.__file__.rsplit("/", 1)[0])
    assert out.returncode == 0, out.stderr[-500:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == impl and "unavailable" in line
