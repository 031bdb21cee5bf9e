"""GPU visibility resolution and NVIDIA MPS daemon lifecycle for oversubscribed inference.

No ``torch`` import at module level: this module has to run before any CUDA call, because
``CUDA_VISIBLE_DEVICES`` is read once when the driver library initialises.  Behaviour follows the
reference (opt_prime/opt_prime/mps_manager.py:165-961):

* ``resolve_visible_devices(num_gpus, gpu_ids, use_mps)`` reconciles ``--num-gpus`` / ``--gpu-ids`` with the
  environment (decision table in the docstring), re-``exec``s the process when the visible set has to change
  (the only reliable way), and never touches the variable under MPS (there a mismatch is an error);
* a file barrier with ready / abort sentinels and a time limit lets local ranks agree that the daemon is up;
* ``MPSManager`` starts or re-uses ``nvidia-cuda-mps-control -d``, cleans stale pipe directories, snapshots
  and restores the environment, sets ``NCCL_LAUNCH_MODE=PARALLEL``, and stops the daemon it started at exit
  or on SIGINT/SIGTERM.

MPS changes how every process on the GPU is scheduled, so everything here is opt-in (``use_mps=True``) and
the daemon commands go through an injectable runner, which the CPU tests replace by a fake.
"""
from __future__ import annotations

import atexit
import os
import shutil
import signal
import subprocess
import sys
import time
from typing import Callable, Dict, List, Optional

_resolve_snapshot: Dict[str, Optional[str]] = {}
REEXEC_SENTINEL = "_OPT_PRIME_MPS_REEXEC"


def _warn(msg: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(f"[aicomp_b200][MPS] WARNING: {msg}", file=sys.stderr)


def _info(msg: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(f"[aicomp_b200][MPS] {msg}", file=sys.stderr)


class MPSConfigError(RuntimeError):
    pass


def parse_gpu_ids(text: str) -> List[int]:
    ids = []
    for part in text.split(","):
        part = part.strip()
        if not part:
            continue
        if not part.isdigit():
            raise MPSConfigError(f"--gpu-ids must be a comma-separated list of non-negative integers, got {text!r}")
        ids.append(int(part))
    if len(set(ids)) != len(ids):
        raise MPSConfigError(f"--gpu-ids contains duplicates: {text!r}")
    return ids


def physical_gpu_count(runner: Optional[Callable[[List[str]], str]] = None) -> int:
    """Number of GPUs nvidia-smi lists (independent of CUDA_VISIBLE_DEVICES); 0 when it cannot be asked."""
    try:
        out = (runner or _run)(["nvidia-smi", "--query-gpu=index", "--format=csv,noheader"])
        return len([l for l in out.splitlines() if l.strip()])
    except Exception:
        return 0


def _run(cmd: List[str], input_text: Optional[str] = None) -> str:
    return subprocess.run(cmd, input=input_text, capture_output=True, text=True, timeout=30, check=True).stdout


def resolve_visible_devices(num_gpus: Optional[int], gpu_ids: Optional[str], use_mps: bool = False, reexec: bool = True,
                            runner: Optional[Callable[[List[str]], str]] = None) -> Optional[str]:
    """Reconcile the command line with ``CUDA_VISIBLE_DEVICES``; returns the value that is in force afterwards.

      env CVD | --gpu-ids        | --num-gpus       | action
      --------+------------------+------------------+--------------------------------
      unset   | unset            | unset            | nothing
      unset   | "0,2,4"          | -                | CVD = "0,2,4"
      unset   | -                | N                | CVD = "0,...,N-1"
      set     | unset            | unset            | keep
      set     | same as CVD      | -                | keep
      set     | differs          | -                | override (warning); error under MPS
      set     | -                | same count       | keep
      set     | -                | other count      | override (warning); error under MPS

    ``--gpu-ids`` wins over ``--num-gpus``.  A change of the variable re-executes the interpreter (``reexec``)
    so that the driver sees it from process start; the previous value is kept for ``restore_visible_devices``.
    """
    env_cvd = os.environ.get("CUDA_VISIBLE_DEVICES")
    if num_gpus is not None and gpu_ids is not None:
        _warn("both --num-gpus and --gpu-ids given; using --gpu-ids")
        num_gpus = None
    ids = parse_gpu_ids(gpu_ids) if gpu_ids is not None else None
    if gpu_ids is not None and not ids:
        raise MPSConfigError("--gpu-ids is empty")
    if num_gpus is not None and num_gpus <= 0:
        raise MPSConfigError(f"--num-gpus must be positive, got {num_gpus}")
    phys = physical_gpu_count(runner)
    if phys:
        if ids is not None and any(g >= phys for g in ids):
            raise MPSConfigError(f"--gpu-ids {ids} out of range: this node has {phys} GPUs")
        if num_gpus is not None and num_gpus > phys:
            raise MPSConfigError(f"--num-gpus {num_gpus} exceeds the {phys} GPUs of this node")
    want: Optional[str] = None
    if ids is not None:
        want = ",".join(map(str, ids))
    elif num_gpus is not None:
        if env_cvd is not None and len([x for x in env_cvd.split(",") if x.strip()]) == num_gpus:
            want = env_cvd
        else:
            want = ",".join(map(str, range(num_gpus)))
    if want is None or want == env_cvd:
        return env_cvd
    if use_mps:
        raise MPSConfigError(f"under MPS CUDA_VISIBLE_DEVICES must be set in the shell before launch: environment has "
                             f"{env_cvd!r}, arguments ask for {want!r}")
    if env_cvd is not None:
        _warn(f"overriding CUDA_VISIBLE_DEVICES={env_cvd!r} with {want!r}")
    _resolve_snapshot.setdefault("CUDA_VISIBLE_DEVICES", env_cvd)
    os.environ["CUDA_VISIBLE_DEVICES"] = want
    if reexec and "torch" in sys.modules and getattr(sys.modules["torch"], "cuda", None) is not None \
            and sys.modules["torch"].cuda.is_initialized():
        _warn("CUDA is already initialised in this process; the new device set takes effect only after re-exec")
    if reexec and os.environ.get(REEXEC_SENTINEL) is None:
        os.environ[REEXEC_SENTINEL] = "1"
        sys.stdout.flush()
        sys.stderr.flush()
        os.execv(sys.executable, [sys.executable] + sys.argv)
    return want


def restore_visible_devices() -> None:
    if "CUDA_VISIBLE_DEVICES" in _resolve_snapshot:
        old = _resolve_snapshot.pop("CUDA_VISIBLE_DEVICES")
        if old is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES", None)
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = old


# ---------------------------------------------------------------- file barrier between local ranks
class FileBarrier:
    """``ready`` / ``abort`` sentinel files in a shared directory; waiters give up after ``timeout_s``."""

    def __init__(self, directory: str, timeout_s: float = 60.0):
        self.dir = directory
        self.timeout_s = timeout_s
        os.makedirs(directory, exist_ok=True)

    def _p(self, name: str) -> str:
        return os.path.join(self.dir, name)

    def signal_ready(self) -> None:
        open(self._p("ready"), "w").close()

    def signal_abort(self, reason: str = "") -> None:
        with open(self._p("abort"), "w") as f:
            f.write(reason)

    def wait(self) -> None:
        t0 = time.time()
        while time.time() - t0 < self.timeout_s:
            if os.path.exists(self._p("abort")):
                raise RuntimeError("MPS set-up aborted by the leader: " + open(self._p("abort")).read())
            if os.path.exists(self._p("ready")):
                return
            time.sleep(0.05)
        raise TimeoutError(f"no ready signal in {self.dir} within {self.timeout_s}s")

    def clear(self) -> None:
        for n in ("ready", "abort"):
            try:
                os.remove(self._p(n))
            except FileNotFoundError:
                pass


# ---------------------------------------------------------------- daemon lifecycle
class MPSManager:
    ENV_KEYS = ("CUDA_MPS_PIPE_DIRECTORY", "CUDA_MPS_LOG_DIRECTORY", "NCCL_LAUNCH_MODE", "CUDA_MPS_ACTIVE_THREAD_PERCENTAGE")

    def __init__(self, pipe_dir: str = "/tmp/nvidia-mps", log_dir: str = "/tmp/nvidia-mps-log", thread_percentage: Optional[int] = None,
                 runner: Optional[Callable[..., str]] = None, register_handlers: bool = True):
        self.pipe_dir, self.log_dir = pipe_dir, log_dir
        self.thread_percentage = thread_percentage
        self._run = runner or _run
        self.started_by_us = False
        self._env_snapshot: Dict[str, Optional[str]] = {}
        self._register = register_handlers
        self._old_handlers = {}

    def is_running(self) -> bool:
        try:
            out = self._run(["pgrep", "-x", "nvidia-cuda-mps-control"])
            return bool(out.strip())
        except Exception:
            return False

    def _apply_env(self) -> None:
        new = {"CUDA_MPS_PIPE_DIRECTORY": self.pipe_dir, "CUDA_MPS_LOG_DIRECTORY": self.log_dir, "NCCL_LAUNCH_MODE": "PARALLEL"}
        if self.thread_percentage is not None:
            new["CUDA_MPS_ACTIVE_THREAD_PERCENTAGE"] = str(self.thread_percentage)
        for k in self.ENV_KEYS:
            self._env_snapshot.setdefault(k, os.environ.get(k))
        os.environ.update(new)

    def restore_env(self) -> None:
        for k, v in self._env_snapshot.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
        self._env_snapshot.clear()

    def _cleanup_stale(self) -> None:
        """A pipe directory without a live daemon is left over from a crashed run."""
        if os.path.isdir(self.pipe_dir) and not self.is_running():
            shutil.rmtree(self.pipe_dir, ignore_errors=True)

    def start(self) -> bool:
        """Start the daemon unless one is running; returns True when this call started it."""
        self._apply_env()
        if self.is_running():
            _info("re-using the running MPS control daemon")
            return False
        self._cleanup_stale()
        os.makedirs(self.pipe_dir, exist_ok=True)
        os.makedirs(self.log_dir, exist_ok=True)
        self._run(["nvidia-cuda-mps-control", "-d"])
        self.started_by_us = True
        if self._register:
            atexit.register(self.stop)
            for sig in (signal.SIGINT, signal.SIGTERM):
                try:
                    self._old_handlers[sig] = signal.signal(sig, self._on_signal)
                except ValueError:
                    pass  # not in the main thread
        return True

    def _on_signal(self, signum, frame):
        self.stop()
        old = self._old_handlers.get(signum)
        if callable(old):
            old(signum, frame)
        else:
            raise SystemExit(128 + signum)

    def stop(self) -> None:
        if self.started_by_us:
            try:
                self._run(["nvidia-cuda-mps-control"], "quit\n")
            except Exception:
                pass
            self.started_by_us = False
        self.restore_env()


def setup_mps_for_inference(use_mps: bool, num_gpus: Optional[int] = None, gpu_ids: Optional[str] = None,
                            barrier_dir: Optional[str] = None, runner=None) -> Optional[MPSManager]:
    """What an inference script calls first: resolve devices; with ``use_mps`` local rank 0 brings the daemon up and the
    other local ranks wait on the file barrier."""
    resolve_visible_devices(num_gpus, gpu_ids, use_mps, runner=runner)
    if not use_mps:
        return None
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    barrier = FileBarrier(barrier_dir or f"/tmp/aicomp_mps_barrier_{os.environ.get('MASTER_PORT', '0')}")
    mgr = MPSManager(runner=runner)
    if local_rank == 0:
        barrier.clear()
        try:
            mgr.start()
            barrier.signal_ready()
        except Exception as e:
            barrier.signal_abort(repr(e))
            raise
    else:
        mgr._apply_env()
        barrier.wait()
    return mgr
