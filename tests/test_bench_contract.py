"""CPU tests of `bench.py` pieces that do not need a GPU: the clock sampler (against a fake
`nvidia-smi` on PATH), the config block of the JSON line and the reference arm's `unavailable` answer."""
import importlib.util
import json
import os
import stat
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


FAKE_SMI = """#!/usr/bin/env python3
import sys, time
loop = "-lms" in sys.argv
n = 0
while True:
    sm = 1500 + 10 * n
    print(f"{sm}, 1965, 700.0, Not Active, Not Active, Not Active, Active", flush=True)
    n += 1
    if not loop:
        break
    time.sleep(0.05)
"""


def test_clock_sampler_uses_one_process_and_only_samples_of_the_timed_region(tmp_path, monkeypatch):
    fake = tmp_path / "nvidia-smi"
    fake.write_text(FAKE_SMI)
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    bench = _load_bench()
    s = bench.ClockSampler(0)
    s.start()                       # before the "warm-up"
    time.sleep(0.4)
    pid = s._p.pid
    s.begin()                       # timed region starts: earlier samples must not count
    time.sleep(0.5)
    out = s.stop()
    assert s._p.pid == pid and s._p.poll() is not None          # one process, ended by its handle
    assert out["sm_max_mhz"] == 1965.0 and out["reasons"] == ["sw_power_cap"]
    assert 3 <= out["samples"] <= 14
    # the fake raises its clock with every sample: the samples of the first 0.4 s (< 1 550 MHz) are gone
    assert out["sm_mhz"] >= 1550.0


def test_clock_sampler_without_nvidia_smi_reports_no_samples(tmp_path, monkeypatch):
    monkeypatch.setenv("PATH", str(tmp_path))            # nothing on PATH
    bench = _load_bench()
    s = bench.ClockSampler(0)
    s.start()
    s.begin()
    out = s.stop()
    assert out["samples"] == 0 and out["sm_mhz"] is None


def test_config_block_names_the_benchmark_configuration():
    bench = _load_bench()
    cfg = bench.config_block(8, 2)
    assert cfg["global_batch"] == 1048576 and cfg["seq_len"] == 512
    assert cfg["parallelism"].startswith("dp8") and cfg["grad_accum"] == 2
    assert "l2_policy" in cfg and "padding_tail" in cfg
    json.dumps(cfg)


def test_reference_arm_answers_unavailable_without_the_installed_reference(tmp_path):
    """A copy of bench.py next to no `baseline/_ref` prints the one-line unavailable record and exits 0."""
    work = tmp_path / "repo"
    work.mkdir()
    (work / "bench.py").write_text((ROOT / "bench.py").read_text())
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    r = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--steps", "1", "--warmup", "3"],
                       cwd=work, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-400:]
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    rec = json.loads(line)
    assert rec["impl"] == "reference" and "unavailable" in rec


def test_data_bench_runs_both_arms(tmp_path):
    """The host data pipeline benchmark prints one JSON line per measurement for this package and,
    when the reference is installed under baseline/_ref, for the reference's classes on the same shards."""
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, PYTHONPATH=str(root), CUDA_VISIBLE_DEVICES="")
    arms = ["own"] + (["reference"] if (root / "baseline" / "_ref" / "nanoplm").exists() else [])
    for arm in arms:
        out = subprocess.run([sys.executable, "-m", "nanoplm_b200.bench.data_bench", "--sequences", "600", "--batch", "52",
                              "--rows", "32", "--workers", "0", "--impl", arm], cwd=tmp_path, env=env,
                             capture_output=True, text=True, timeout=600)
        assert out.returncode == 0, (out.stdout + out.stderr)[-3000:]
        rows = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
        names = [r["bench"] for r in rows]
        for want in ("read_every_sequence", "tokenize_one_by_one", "packing_collator_static", "padding_collator"):
            assert want in names, (arm, names)
        assert all(r.get("impl", arm) == arm for r in rows)
        static = next(r for r in rows if r["bench"] == "packing_collator_static")
        assert static["real_tokens_per_s"] > 0 and static["micro_batches"] >= 5
