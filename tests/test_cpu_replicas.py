"""The N > 1 path of the benchmark on CPU: two gloo ranks, the barrier, the
max-over-ranks time and the whole-job rate (replicas only, no data-path collective)."""
import os
import socket
import subprocess
import sys
import textwrap
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]

WORKER = textwrap.dedent("""
    import json, sys
    sys.path.insert(0, sys.argv[1])
    from clpeak_b200.replicas import Replicas
    r = Replicas("gloo")
    assert r.active and r.world == 2
    r.barrier()
    r.host_barrier()                                   # the CPU-only wait used while one rank drives every GPU
    local_ms = 10.0 if r.rank == 0 else 25.0          # rank 1 is the slow replica
    rate, ms = r.whole_job_rate(1000.0, local_ms)
    mx = r.max_over_ranks(float(r.rank))
    print(json.dumps({"rank": r.rank, "rate": rate, "ms": ms, "mx": mx, "local_world": r.local_world}), flush=True)
    r.close()
""")


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_gloo_replicas_agree_on_the_slowest_time(tmp_path):
    import json
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE="2",
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script), str(ROOT)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        out, err = p.communicate(timeout=180)
        assert p.returncode == 0, err[-2000:]
        outs.append(json.loads(out.strip().splitlines()[-1]))
    for o in outs:
        assert o["ms"] == 25.0                       # every rank divides by the slowest replica's time
        assert abs(o["rate"] - 2 * 1000.0 / 0.025) < 1e-6
        assert o["mx"] == 1.0 and o["local_world"] == 2
    assert sorted(o["rank"] for o in outs) == [0, 1]


def test_single_replica_needs_no_process_group(monkeypatch):
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE"):
        monkeypatch.delenv(k, raising=False)
    sys.path.insert(0, str(ROOT))
    from clpeak_b200.replicas import Replicas
    r = Replicas("gloo")
    assert not r.active and r.world == 1 and r.rank == 0
    r.barrier()
    r.host_barrier()
    rate, ms = r.whole_job_rate(500.0, 5.0)
    assert ms == 5.0 and rate == 500.0 / 0.005
    r.close()
