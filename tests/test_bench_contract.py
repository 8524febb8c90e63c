"""bench.py's reference arm on its CPU-sized workload: the line it prints has the keys the benchmark contract asks
for, describes the workload with the same `config` keys as the GPU arm, never loads the product library, and a run
that does not finish within --deadline ends with exit code 124."""
import ast
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "bench.py")


def _run(*extra, timeout=600):
    return subprocess.run([sys.executable, BENCH, *extra], capture_output=True, text=True, timeout=timeout, cwd=ROOT,
                          stdin=subprocess.DEVNULL)


def test_reference_arm_line():
    proc = _run("--impl", "reference", "--workload", "gcn_c1", "--steps", "2", "--warmup", "1")
    assert proc.returncode == 0, proc.stderr[-500:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["metric"] == "gcn_epoch_ms" and line["unit"] == "ms"
    assert line["steps"] == 2 and line["warmup"] == 1 and line["n_gpus"] == 1 and line["higher_is_better"] is False
    assert line["value"] > 0 and line["value"] == line["ms_per_step"] == line["e2e"]["value"] == line["cpu_baseline"]["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1 and line["cpu_baseline"]["sample"]
    assert line["config"]["workload"] == "gcn_c1" and line["config"]["nodes"] == 19717
    assert line["gpu_launches"] == 0


def test_both_arms_describe_the_workload_with_the_same_config_keys():
    """The `config` dict literals of run_ours and run_reference have identical keys (the GPU arm cannot run here, so
    this reads the source)."""
    tree = ast.parse(open(BENCH).read())
    keys = {}
    for fn in tree.body:
        if isinstance(fn, ast.FunctionDef) and fn.name in ("run_ours", "run_reference"):
            for node in ast.walk(fn):
                if isinstance(node, ast.Dict):
                    for k, v in zip(node.keys, node.values):
                        if isinstance(k, ast.Constant) and k.value == "config" and isinstance(v, ast.Dict):
                            keys[fn.name] = [kk.value for kk in v.keys]
    assert set(keys) == {"run_ours", "run_reference"}
    assert keys["run_ours"] == keys["run_reference"] == ["workload", "nodes", "edges", "layers", "timing"]


def test_reference_arm_does_not_load_the_product_library():
    code = ("import sys, types; sys.argv=['bench.py']; import bench\n"
            "ns = types.SimpleNamespace(workload='gcn_c1', steps=1, warmup=0, gpus=1)\n"
            "bench.run_reference(ns)\n"
            "assert not any(m.startswith('tango_b200._lib') or m == 'tango_b200.kernels' for m in sys.modules), 'package binding imported'\n"
            "assert 'libtango_b200' not in open('/proc/self/maps').read(), 'product library mapped'\n")
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-800:]


def test_deadline_ends_a_run_that_does_not_finish():
    proc = _run("--impl", "reference", "--workload", "gcn_c1", "--steps", "100000", "--warmup", "0", "--deadline", "3",
                timeout=120)
    assert proc.returncode == 124 and "giving up" in proc.stderr
