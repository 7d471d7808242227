"""The JSON line bench.py prints (checked here without a GPU) and its reference-arm fall-back."""
import argparse
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_json_line_has_the_contract_fields(capsys):
    bench = _bench()
    args = argparse.Namespace(steps=20, warmup=5, optimizer="dion2")
    clocks = {"sm_mhz": 1700.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"]}
    bench.emit(args, "ours", 700.0, 720.0, clocks, 3380, 2, {"final_loss": 1.0})
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step",
                "higher_is_better", "scaling", "vs_baseline", "dtype", "data", "config", "clocks",
                "gpu_launches", "e2e"):
        assert key in line, key
    assert line["n_gpus"] == 2 and line["steps"] == 20 and line["warmup"] == 5
    assert line["higher_is_better"] is True and line["scaling"] == "weak" and line["dtype"] == "bf16"
    assert line["ms_per_step"] == 35.0
    tokens = 2 * bench.DEVICE_BATCH * bench.SEQ * 20
    assert abs(line["value"] - tokens / 0.7) < 1e-6          # whole-job tokens/s
    assert line["config"]["global_batch"] == 2 * bench.DEVICE_BATCH
    assert line["config"]["seq_len"] == bench.SEQ and line["config"]["parallelism"] == "ddp2"
    assert set(line["e2e"]) >= {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"}
    assert line["e2e"]["h2d_bytes_per_step"] == 2 * bench.DEVICE_BATCH * bench.SEQ * 8
    assert line["gpu_launches"] == 3380


def test_defaults_are_one_gpu_and_a_short_run():
    bench = _bench()
    old = sys.argv
    sys.argv = ["bench.py"]
    try:
        args = bench.parse()
    finally:
        sys.argv = old
    assert args.gpus == 1 and args.impl == "ours" and args.warmup >= 3 and args.steps <= 50


def test_reference_arm_reports_unavailable_when_not_installed(tmp_path):
    """Without baseline/_ref the reference arm prints its `unavailable` line and exits 0."""
    copy = tmp_path / "bench.py"
    copy.write_text(open(os.path.join(ROOT, "bench.py")).read())
    res = subprocess.run([sys.executable, str(copy), "--impl", "reference"], capture_output=True,
                         text=True, timeout=300, cwd=str(tmp_path))
    assert res.returncode == 0, res.stderr[-500:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line


def test_newton_schulz_benchmark_curve_writer(tmp_path, capsys):
    """The size sweep of the Newton-Schulz benchmark writes a CSV and a text chart without a
    plotting library."""
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location(
        "bench_newton_schulz", os.path.join(root, "benchmark", "bench_newton_schulz.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    rows = [{"batch": 1, "m": 128, "n": 128, "a": {"tflops": 10.0}, "b": {"tflops": 5.0}},
            {"batch": 1, "m": 256, "n": 256, "a": {"tflops": 30.0}, "b": {"error": "x"}}]
    path = mod.write_curve(rows, ["a", "b"], str(tmp_path), "curve")
    assert open(path).read().splitlines() == ["dim,a,b", "128,10.0,5.0", "256,30.0,"]
    assert "#" * 50 in capsys.readouterr().out
    assert mod.ns_flops(2, 8, 4) == 2 * 5 * (4.0 * 16 * 8 + 2.0 * 64)


def test_reference_benchmark_command_line_is_translated():
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location(
        "benchmark_newton_shultz", os.path.join(root, "benchmark", "benchmark_newton_shultz.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.translate(["--single", "--m", "1024"]) == ["--batch", "1", "--single", "1024", "1024"]
    assert mod.translate(["--single", "--m", "768", "--n", "3072", "--batch_size", "4"]) == \
        ["--batch", "4", "--single", "768", "3072"]
    assert mod.translate(["--grid", "--expansion", "4"]) == ["--batch", "1", "--sweep", "--expansion", "4"]
    assert mod.translate(["--plot", "--batch_size", "2"]) == ["--batch", "2", "--curve"]


def test_aux_block_work_model():
    """Work of the GPT-1B Muon step used for the roofline fractions of the `aux` block."""
    bench = _bench()
    shapes = bench.aux_shapes()
    assert len(shapes) == 144 and shapes.count((2048, 2048)) == 96
    one = bench.aux_bounds(1)
    eight = bench.aux_bounds(8)
    # 5 x (4 m^2 n + 2 m^3): 96 square matrices + 48 matrices of 2048 x 8192
    nominal = 5 * (96 * 6 * 2048 ** 3 + 48 * (4 * 2048 ** 2 * 8192 + 2 * 2048 ** 3)) / 1e12
    assert abs(one["ns_tflop_nominal_per_gpu"] - nominal) < 1e-6
    assert abs(eight["ns_tflop_nominal_per_gpu"] * 8 - nominal) < 1e-6
    assert one["ns_tflop_needed_per_gpu"] < one["ns_tflop_nominal_per_gpu"]
    assert one["nvlink_mb_sent_per_gpu"] == 0 and one["nvlink_bound_ms"] == 0
    # every rank sends 7/8 of its 1/8 of all bf16 elements, once out and once back
    elems = 96 * 2048 ** 2 + 48 * 2048 * 8192
    assert abs(eight["nvlink_mb_sent_per_gpu"] - 2 * elems * 2 / 8 * 7 / 8 / 1e6) < 1e-6
    assert eight["roofline_ms"] == max(eight["compute_bound_ms"], eight["nvlink_bound_ms"])
