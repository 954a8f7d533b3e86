"""The benchmark's reference arm runs on the host cores alone: its JSON line carries the keys the contract names,
and the helpers that label and pick peaks behave as documented (no GPU needed)."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_one_contract_line():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in line, key
    assert line["impl"] == "reference" and line["metric"] == "moe_layer_fwd_bwd_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["vs_baseline"] is None and line["gpu_launches"] == 0
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and "sample" in cb
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in line["config"]


def test_parallelism_label_names_the_data_plane(monkeypatch):
    b = _bench()
    assert b._parallelism_label(1) == "single GPU"
    monkeypatch.delenv("B200MOE_EP_TRANSPORT", raising=False)
    monkeypatch.delenv("B200MOE_EP_EXCHANGE", raising=False)
    monkeypatch.delenv("B200MOE_EP_CAPACITY", raising=False)
    label = b._parallelism_label(8)
    assert "transport=p2p" in label and "exchange=push" in label and "fixed capacity" in label and "1.5" in label
    monkeypatch.setenv("B200MOE_EP_CAPACITY", "0")
    assert "fixed capacity" not in b._parallelism_label(8)
    monkeypatch.setenv("B200MOE_EP_TRANSPORT", "nccl")
    assert "all_to_all_single" in b._parallelism_label(2)


def test_roofline_denominator_follows_the_sampled_clock():
    """The fraction is taken against the burst figure only when the timed region ran at >= 90 % of the maximum SM
    clock, against the sustained figure otherwise; both fractions are always printed."""
    b = _bench()
    peaks = dict(burst=1689.0, sustained=1434.2)
    assert b._pick_peak(peaks, {"sm_mhz": 1950.0, "sm_max_mhz": 1965.0}) == ("burst", 1689.0)
    assert b._pick_peak(peaks, {"sm_mhz": 1768.5, "sm_max_mhz": 1965.0}) == ("burst", 1689.0)      # exactly 90 %
    assert b._pick_peak(peaks, {"sm_mhz": 1432.0, "sm_max_mhz": 1965.0}) == ("sustained", 1434.2)
    assert b._pick_peak(peaks, None)[1] == 1434.2 and b._pick_peak(peaks, {})[0].startswith("sustained")
    f = b._fractions(1000.0, peaks, {"sm_mhz": 1432.0, "sm_max_mhz": 1965.0})
    assert f["rule"] == "sustained" and f["peak"] == 1434.2 and f["frac"] == f["frac_of_sustained"] == round(1000 / 1434.2, 4)
    assert f["frac_of_burst"] == round(1000 / 1689.0, 4)
    fp8 = b._peaks("mxfp8")
    bf = b._peaks("bf16")
    assert fp8["burst"] == 2 * bf["burst"] and fp8["sustained"] == 2 * bf["sustained"] and fp8["source"].startswith("2 x")
