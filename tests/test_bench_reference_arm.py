"""The CPU arm of bench.py (`--impl reference`: the C restatement of the reference's decode step timed on the host cores), launched
the way a multi-GPU run launches it: two workers under torch.distributed.run.  Rank 0 alone prints the line, the other rank exits
0 without work, the line carries the benchmark's metric string, and the arm uses all the host cores although the launcher exports
OMP_NUM_THREADS=1 to its workers."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_under_the_distributed_launcher():
    env = dict(os.environ)
    env.pop("OMP_NUM_THREADS", None)
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                          "--master-port", "29541", os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, res.stdout
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2 and d["steps"] == 2 and d["warmup"] == 1
    assert d["metric"] == "decode tokens/s (Llama-2-7B INT4 g128, batch 1, prompt 512)" and d["unit"] == "tokens/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["cpu_baseline"]["kind"] == "port" and d["e2e"]["h2d_bytes_per_step"] == 0
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count()
    assert d["cpu_baseline"]["cores"] == cores
