"""The parts of the root benchmark script that can be checked without a GPU: its arguments, the configurations
it names, its FLOP count against the model's own, and the ``unavailable`` line it prints when no GPU is there."""
import importlib.util
import json
import pathlib
import subprocess
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("bench_script", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("impl", ["ours", "reference"])
def test_without_a_gpu_the_script_says_so_in_one_json_line(impl):
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", impl], capture_output=True, text=True,
                         timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == impl and "unavailable" in line


def test_flop_count_matches_the_model_and_meshes_multiply_out():
    import forgeminds_b200 as fm
    b = _bench()
    assert set(b.CONFIGS) == {"dense", "moe", "llama8b", "gpt2p7b"}
    spec = b.CONFIGS["dense"]
    model = fm.GPT(fm.GPTConfig(ffn_hidden=spec["hidden"], **{**spec["model"], "n_layers": 2}))
    two_layers = dict(spec, model={**spec["model"], "n_layers": 2})
    assert b.full_model_flops_per_token(two_layers, False) == model.flops_per_token(spec["seq"])
    for name, world in (("dense", 8), ("moe", 8), ("llama8b", 8), ("gpt2p7b", 8), ("llama8b", 4), ("gpt2p7b", 2)):
        mesh = b.CONFIGS[name]["mesh"](world)
        size = 1
        for key in ("dp_replicate", "dp_shard", "tp", "pp"):
            size *= mesh.get(key, 1)
        assert size == world, (name, world, mesh)
        assert world % b.CONFIGS[name].get("min_world", 1) == 0


def test_cpu_configuration_runs_through_the_public_trainer():
    """``--config tiny`` is the baseline list's CPU / Gloo configuration: one process here, two steps."""
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--config", "tiny", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert line["device"] == "cpu" and line["dtype"] == "fp32" and line["impl"] == "ours"
    assert line["value"] > 0 and line["config"]["seq_len"] == 256 and 9.0 < line["final_loss"] < 11.5
