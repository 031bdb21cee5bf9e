"""Multi-process test harness: N local ranks over gloo (or NCCL), with a timeout.

Pattern of the reference's ``@distributed_test`` decorator (gpt-neox/tests/common.py:128-238):
fork N processes on one node, rendezvous on 127.0.0.1, join with a timeout, and turn a
hang, a signal or a non-zero exit into a test failure.  Ranks here are fresh interpreter
processes running ``tests/workers/<name>.py``; each writes its result as JSON.
"""
import json
import os
import socket
import subprocess
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_workers(worker: str, world_size: int, args=None, timeout: float = 240.0, env_extra=None, expect_fail_ranks=()):
    """Run ``tests/workers/<worker>.py`` on ``world_size`` ranks; returns the list of per-rank result dicts."""
    port = free_port()
    outdir = tempfile.mkdtemp(prefix=f"aicomp_{worker}_")
    procs = []
    for rank in range(world_size):
        env = dict(os.environ)
        env.update({"RANK": str(rank), "WORLD_SIZE": str(world_size), "LOCAL_RANK": str(rank), "LOCAL_WORLD_SIZE": str(world_size),
                    "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "AICOMP_TEST_OUT": outdir,
                    "PYTHONPATH": REPO + os.pathsep + env.get("PYTHONPATH", ""), "OMP_NUM_THREADS": "2",
                    "AICOMP_TEST_ARGS": json.dumps(args or {})})
        env.update(env_extra or {})
        log = open(os.path.join(outdir, f"rank{rank}.log"), "w")
        p = subprocess.Popen([sys.executable, os.path.join(REPO, "tests", "workers", worker + ".py")], env=env, stdout=log,
                             stderr=subprocess.STDOUT, start_new_session=True)
        procs.append((p, log))
    deadline = time.time() + timeout
    failed = None
    for rank, (p, log) in enumerate(procs):
        try:
            rc = p.wait(timeout=max(1.0, deadline - time.time()))
        except subprocess.TimeoutExpired:
            failed = f"rank {rank} timed out after {timeout}s"
            break
        if rc != 0 and rank not in expect_fail_ranks:
            failed = f"rank {rank} exited with {rc}"
            break
    if failed:
        for p, _ in procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, 9)
                except ProcessLookupError:
                    pass
    for _, log in procs:
        log.close()
    if failed:
        tails = []
        for rank in range(world_size):
            with open(os.path.join(outdir, f"rank{rank}.log")) as f:
                tails.append(f"--- rank {rank} ---\n" + "".join(f.readlines()[-25:]))
        raise AssertionError(failed + "\n" + "\n".join(tails))
    results = []
    for rank in range(world_size):
        path = os.path.join(outdir, f"rank{rank}.json")
        results.append(json.load(open(path)) if os.path.exists(path) else None)
    return results


def worker_args():
    return json.loads(os.environ.get("AICOMP_TEST_ARGS", "{}"))


def worker_report(obj) -> None:
    out = os.environ["AICOMP_TEST_OUT"]
    with open(os.path.join(out, f"rank{os.environ['RANK']}.json"), "w") as f:
        json.dump(obj, f)
