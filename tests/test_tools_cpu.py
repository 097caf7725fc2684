"""Autotune, the command-line tools and the DeepSpeed config builder, all on CPU with fake workloads."""
import json
import subprocess
import sys
import time

import pytest
import torch

import forgeminds_b200 as fm


# ------------------------------------------------------------------ autotune
def test_time_call_is_a_median_after_warmup():
    from forgeminds_b200.autotune import time_call
    calls = []

    def fn():
        calls.append(time.perf_counter())
        time.sleep(0.002)

    ms = time_call(fn, warmup=2, repeats=3, sync=False)
    assert len(calls) == 5 and 1.5 < ms < 50


def test_tune_batch_size_treats_out_of_memory_as_data():
    from forgeminds_b200.autotune import Report, tune_batch_size
    seen = []

    def step(size):
        seen.append(size)
        if size >= 16:
            raise RuntimeError("CUDA out of memory. Tried to allocate 1 GiB")
        time.sleep(0.001 * (1 + 0.25 * size))          # cost per sample keeps falling

    rep = Report()
    size, ms = tune_batch_size(step, candidates=(1, 2, 4, 8, 16, 32), warmup=0, repeats=2, report=rep)
    assert size == 8 and ms < float("inf")
    assert 32 not in seen                               # stopped at the first size that did not fit
    assert any(t.oom for t in rep.trials)
    assert "micro_batch=16" in rep.table()


def test_tune_batch_size_stops_without_gain_and_reraises_other_errors():
    from forgeminds_b200.autotune import tune_batch_size

    def flat(size):
        time.sleep(0.002 * size)                        # no gain per sample from batching

    size, _ = tune_batch_size(flat, candidates=(1, 2, 4), warmup=0, repeats=2, min_gain=0.2)
    assert size == 1

    def broken(size):
        raise ValueError("not an allocation problem")

    with pytest.raises(ValueError):
        tune_batch_size(broken, candidates=(1, 2))


def test_apply_fast_defaults_reports_what_it_set():
    from forgeminds_b200.autotune import apply_fast_defaults
    out = apply_fast_defaults(device=torch.device("cpu"))
    assert isinstance(out, dict)


# ------------------------------------------------------------------ command line
def _cli(*args, timeout=300):
    return subprocess.run([sys.executable, "-m", "forgeminds_b200.cli", *args], capture_output=True, text=True,
                          timeout=timeout)


def test_kbench_check_refuses_to_judge_without_a_gpu():
    if torch.cuda.is_available():
        pytest.skip("needs a machine without CUDA")
    out = _cli("kbench", "--check", "--ops", "rms_norm")
    assert out.returncode == 2, out.stderr[-2000:]


def test_kbench_runs_on_cpu_when_allowed(tmp_path):
    if torch.cuda.is_available():
        pytest.skip("needs a machine without CUDA")
    target = tmp_path / "k.json"
    out = _cli("kbench", "--allow-cpu", "--ops", "rms_norm,swiglu,softmax,topk", "--tokens", "64", "--dim", "64",
               "--hidden", "128", "--vocab", "512", "--iters", "2", "--warmup", "1", "--dtype", "fp32", "--json",
               str(target))
    assert out.returncode == 0, out.stderr[-2000:]
    rows = json.loads(target.read_text())["rows"]
    assert {r["op"] for r in rows} == {"rms_norm", "swiglu", "softmax", "topk"}


def test_bench_cli_trains_a_tiny_model_on_cpu(tmp_path):
    target = tmp_path / "b.json"
    out = _cli("bench", "--preset", "tiny", "--seq", "32", "--micro-batch", "2", "--steps", "3", "--warmup", "1",
               "--no-prefetch", "--json", str(target))
    assert out.returncode == 0, out.stderr[-3000:]
    rep = json.loads(target.read_text())
    assert rep["tok_s"] > 0 and rep["step_ms_p50"] > 0 and rep["preset"] == "tiny" and rep["engine"] == "library"


def test_audit_cli_counts_host_reads(tmp_path):
    target = tmp_path / "a.json"
    out = _cli("audit", "--preset", "tiny", "--seq", "32", "--micro-batch", "2", "--steps", "3", "--warmup", "1",
               "--no-prefetch", "--json", str(target))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    rep = json.loads(target.read_text())
    assert rep["host_reads_per_step"] <= 1.0 and rep["engine"] == "library"


def test_unknown_subcommand_is_an_error():
    out = _cli("no-such-tool")
    assert out.returncode != 0


# ------------------------------------------------------------------ DeepSpeed config (library optional)
def test_ds_config_rules():
    from forgeminds_b200.parallel.deepspeed_backend import build_ds_config
    cfg = fm.ForgeConfig()
    cfg.parallel.backend, cfg.parallel.zero_stage = "deepspeed", 2
    cfg.train.grad_accum, cfg.train.grad_clip, cfg.train.bf16 = 4, 0.5, True
    ds = build_ds_config(cfg, world=8, micro_batch=2)
    assert ds["train_batch_size"] == 2 * 4 * 8 and ds["gradient_clipping"] == 0.5
    assert ds["zero_optimization"]["stage"] == 2 and ds["bf16"]["enabled"]
    cfg.parallel.tp = 2
    ds = build_ds_config(cfg, world=8, micro_batch=2)
    assert ds["tensor_parallel"]["autotp_size"] == 2 and ds["train_batch_size"] == 2 * 4 * 4
    cfg.parallel.zero_offload_param = True
    with pytest.raises(ValueError):
        build_ds_config(cfg, world=8, micro_batch=2)                 # parameter offload needs stage 3
    cfg.parallel.zero_stage = 3
    assert "offload_param" in build_ds_config(cfg, world=8, micro_batch=2)["zero_optimization"]
    cfg.parallel.pp, cfg.parallel.tp = 2, 1
    with pytest.raises(ValueError):
        build_ds_config(cfg, world=8, micro_batch=2)                 # pipeline stages need stage <= 1


def test_deepspeed_engine_needs_the_library():
    from forgeminds_b200.parallel import deepspeed_backend as ds
    try:
        import deepspeed  # noqa: F401
        pytest.skip("deepspeed is installed")
    except ImportError:
        pass
    with pytest.raises((ImportError, RuntimeError)):
        ds._deepspeed()


def test_gemmbench_is_registered_and_refuses_to_run_without_a_gpu(capsys):
    import torch
    from forgeminds_b200.cli import __main__ as cli
    from forgeminds_b200.cli import gemmbench
    assert "gemmbench" in cli.TOOLS
    if not torch.cuda.is_available():
        assert gemmbench.main([]) == 1
        assert "needs a GPU" in capsys.readouterr().out


# ------------------------------------------------------------------ compile check and probe
PTXAS_SAMPLE = """
ptxas info    : Compiling entry function '_ZN3fmb6kern_aEv' for 'sm_100a'
ptxas info    : Function properties for _ZN3fmb6kern_aEv
    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads
ptxas info    : Used 40 registers, used 1 barriers, 1024 bytes smem
ptxas info    : Compiling entry function '_ZN3fmb6kern_bEv' for 'sm_100a'
ptxas info    : Function properties for _ZN3fmb6kern_bEv
    800 bytes stack frame, 640 bytes spill stores, 700 bytes spill loads
ptxas info    : Used 255 registers, used 0 barriers
"""


def test_compilecheck_reads_the_assembler_report_and_flags_spills():
    from forgeminds_b200.cli import compilecheck as cc
    rows = cc.parse_ptxas(PTXAS_SAMPLE)
    assert [r["registers"] for r in rows] == [40, 255]
    assert rows[0]["smem"] == 1024 and rows[0]["barriers"] == 1 and rows[0]["spill_stores"] == 0
    assert rows[1]["stack"] == 800 and rows[1]["spill_stores"] == 640 and rows[1]["spill_loads"] == 700
    for r, name in zip(rows, cc.demangle([r["name"] for r in rows])):
        r["pretty"] = name
    assert "kern_a" in rows[0]["pretty"]
    bad = cc.problems(rows, max_spill=512)
    assert len(bad) == 1 and "kern_b" in bad[0]
    assert cc.problems(rows, max_spill=2000) == [] and len(cc.warnings(rows, max_spill=2000)) == 1


def test_probe_runs_every_case_on_cpu():
    from forgeminds_b200.cli import probe
    rows = probe.run(torch.device("cpu"), torch.float32)
    assert len(rows) >= 10 and all(r["ok"] for r in rows), [r for r in rows if not r["ok"]]
    assert probe.main(["--device", "cpu", "--json"]) == 0
