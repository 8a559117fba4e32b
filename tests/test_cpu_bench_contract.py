"""``bench.py`` without a GPU: the command-line contract (defaults, warm-up count), the clock sampler against a stand-in
for NVML (read-only queries: nothing is ever set), the physical GPU index under ``CUDA_VISIBLE_DEVICES``, and what both
arms print when no CUDA device is visible."""

import importlib.util
import json
import os
import subprocess
import sys
import time
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_defaults_are_one_gpu_and_enough_warmup(monkeypatch):
    bench = _bench()
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    args = bench.parse_args()
    assert args.gpus == 1 and args.steps >= 1 and args.warmup >= 3 and args.impl == "ours"
    assert args.parallelism == "dp" and args.prompt_shard == "off" and not args.skip_ops
    assert not (args.dev_layers or args.dev_group or args.dev_micro_group or args.dev_no_overlap or args.dev_layers_per_bucket)


def test_clock_sampler_reads_clocks_and_reasons_and_sets_nothing(monkeypatch):
    calls = []
    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    for bit, name in enumerate(("HwSlowdown", "HwThermalSlowdown", "SwThermalSlowdown", "SwPowerCap", "HwPowerBrakeSlowdown")):
        setattr(fake, "nvmlClocksThrottleReason" + name, 1 << bit)
    fake.nvmlInit = lambda: calls.append("init")
    fake.nvmlDeviceGetHandleByIndex = lambda i: ("handle", i)
    fake.nvmlDeviceGetMaxClockInfo = lambda h, kind: 1965
    clock = iter([1400, 1410, 1390] + [1400] * 1000)
    fake.nvmlDeviceGetClockInfo = lambda h, kind: next(clock)
    fake.nvmlDeviceGetCurrentClocksThrottleReasons = lambda h: fake.nvmlClocksThrottleReasonSwPowerCap

    def refuse(name):
        def f(*a, **k):
            raise AssertionError(f"{name} changes a GPU setting")
        return f

    for setter in ("nvmlDeviceSetGpuLockedClocks", "nvmlDeviceResetGpuLockedClocks", "nvmlDeviceSetPowerManagementLimit",
                   "nvmlDeviceSetPersistenceMode", "nvmlDeviceSetApplicationsClocks"):
        setattr(fake, setter, refuse(setter))
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    bench = _bench()
    with bench.ClockSampler(3) as sampler:
        time.sleep(0.5)
    summary = sampler.summary()
    assert summary["sm_max_mhz"] == 1965 and 1390 <= summary["sm_mhz"] <= 1410
    assert summary["reasons"] == ["sw_power_cap"]


def test_physical_gpu_index_follows_visible_devices(monkeypatch):
    bench = _bench()
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "4,6")
    assert bench.physical_gpu_index(1) == 6
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES")
    assert bench.physical_gpu_index(2) == 2


def _run(*argv):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *argv], capture_output=True, text=True, env=env,
                          timeout=600)


def test_without_a_gpu_our_arm_says_so_and_the_reference_arm_prints_its_unavailable_line():
    import torch

    if torch.cuda.is_available():
        return  # a GPU box runs the real thing
    ours = _run("--steps", "1", "--warmup", "3")
    assert ours.returncode != 0 and "no CUDA device" in ours.stderr and "Traceback" not in ours.stderr
    ref = _run("--impl", "reference", "--steps", "1", "--warmup", "3")
    assert ref.returncode == 0
    lines = [line for line in ref.stdout.splitlines() if line.startswith("{")]
    assert lines, ref.stdout + ref.stderr
    record = json.loads(lines[-1])
    assert record["impl"] == "reference" and "unavailable" in record
