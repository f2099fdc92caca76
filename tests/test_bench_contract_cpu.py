"""Host-side parts of bench.py that need no GPU: the CPU-baseline sample, the reference arm's JSON
line and the workload description."""
import importlib.util
import io
import json
import os
from contextlib import redirect_stdout
from types import SimpleNamespace

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_cpu_baseline_sample_is_bounded_and_described():
    bench = _bench()
    from velox_inferer_b200.stack import StackSpec

    tok_s, cores, sample, step_s = bench.cpu_baseline_sample(StackSpec(), 2048, seconds_target=0.2)
    assert tok_s > 0 and cores >= 1 and step_s > 0
    assert "oracle linear" in sample and "GMAC" in sample


def test_reference_arm_prints_one_line_with_the_contract_keys(monkeypatch):
    bench = _bench()
    real = bench.cpu_baseline_sample
    monkeypatch.setattr(bench, "cpu_baseline_sample", lambda spec, m, seconds_target=12.0, threads=0: real(spec, m, 0.1, threads))
    args = SimpleNamespace(layers=64, workload="prefill", m=2048, warmup=1, steps=2, gpus=2, tp="kernel")
    out = io.StringIO()
    with redirect_stdout(out):
        bench.run_reference(args)
    lines = [l for l in out.getvalue().splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == bench.METRIC and d["unit"] == bench.UNIT
    assert d["n_gpus"] == 2 and d["steps"] == 2 and d["warmup"] == 1 and d["higher_is_better"] is True
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and "model" not in d["config"]
    assert d["vs_baseline"] is None


def test_other_ranks_of_the_reference_arm_print_nothing(monkeypatch):
    bench = _bench()
    monkeypatch.setenv("RANK", "1")
    out = io.StringIO()
    with redirect_stdout(out):
        bench.run_reference(SimpleNamespace(layers=64, workload="prefill", m=2048, warmup=0, steps=1, gpus=2, tp="kernel"))
    assert out.getvalue() == ""
