"""Host-side logic of bench.py that needs no GPU: which batch a run takes, the reference arm's line."""
import json
import subprocess
import sys
from pathlib import Path
from types import SimpleNamespace

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def _args(workload, global_batch=0):
    return SimpleNamespace(workload=workload, global_batch=global_batch)


def test_batch_plan_follows_the_configurations():
    import bench
    # "global batch 1024 sharded over 1/2/4/8 GPUs": fixed total, strong scaling
    for world in (1, 2, 4, 8):
        assert bench.batch_plan(_args("vgg_cifar"), world) == (1024, "strong")
        assert bench.batch_plan(_args("wide_mlp"), world) == (16384, "strong")
    # "Batch 32 ... data-parallel at 1/2/4/8 GPUs": the batch is per GPU, weak scaling
    assert bench.batch_plan(_args("transformer_lm"), 1) == (32, "weak")
    assert bench.batch_plan(_args("transformer_lm"), 8) == (256, "weak")
    # an explicit --global-batch is always a global batch
    assert bench.batch_plan(_args("transformer_lm", 64), 4) == (64, "strong")
    assert bench.batch_plan(_args("vgg_cifar", 128), 1) == (128, "strong")


def test_every_workload_names_a_table_of_the_package():
    import bench
    from neuralrs_b200 import workloads
    for name, (table, batch, _seed, cpu_batch) in bench.WORKLOADS.items():
        cfg = getattr(workloads, table)
        assert cfg["layers"] and batch >= cpu_batch > 0, name


def test_reference_arm_on_other_ranks_prints_nothing():
    # under torchrun only rank 0 runs the CPU arm; the others exit 0 without work
    env = {"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1", "PATH": "/usr/bin:/bin"}
    import os
    env = {**os.environ, **env}
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "1"], env=env, capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr[-500:]
    assert out.stdout.strip() == ""
