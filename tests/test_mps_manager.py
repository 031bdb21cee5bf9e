"""MPS manager on CPU with a fake command runner: no daemon is started, no GPU setting is touched."""
import os

import pytest

from aicomp_b200.utils import mps_manager as mm


class FakeRunner:
    def __init__(self, gpus=8, daemon=False):
        self.gpus, self.daemon, self.calls = gpus, daemon, []

    def __call__(self, cmd, input_text=None):
        self.calls.append((tuple(cmd), input_text))
        if cmd[0] == "nvidia-smi":
            return "\n".join(str(i) for i in range(self.gpus)) + "\n"
        if cmd[0] == "pgrep":
            return "123\n" if self.daemon else ""
        if cmd == ["nvidia-cuda-mps-control", "-d"]:
            self.daemon = True
            return ""
        if cmd == ["nvidia-cuda-mps-control"] and input_text == "quit\n":
            self.daemon = False
            return ""
        raise AssertionError(cmd)


@pytest.fixture(autouse=True)
def clean_env(monkeypatch):
    for k in ("CUDA_VISIBLE_DEVICES", mm.REEXEC_SENTINEL, "CUDA_MPS_PIPE_DIRECTORY", "NCCL_LAUNCH_MODE"):
        monkeypatch.delenv(k, raising=False)
    mm._resolve_snapshot.clear()


def test_decision_table(monkeypatch):
    r = FakeRunner()
    assert mm.resolve_visible_devices(None, None, runner=r, reexec=False) is None
    assert mm.resolve_visible_devices(None, "0,2,4", runner=r, reexec=False) == "0,2,4"
    mm.restore_visible_devices()
    assert "CUDA_VISIBLE_DEVICES" not in os.environ
    assert mm.resolve_visible_devices(3, None, runner=r, reexec=False) == "0,1,2"
    mm.restore_visible_devices()
    # env set, matching count -> kept as is
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "4,5,6")
    assert mm.resolve_visible_devices(3, None, runner=r, reexec=False) == "4,5,6"
    # differing ids -> override; restore brings the old value back
    assert mm.resolve_visible_devices(None, "1,2", runner=r, reexec=False) == "1,2"
    mm.restore_visible_devices()
    assert os.environ["CUDA_VISIBLE_DEVICES"] == "4,5,6"
    with pytest.raises(mm.MPSConfigError):
        mm.resolve_visible_devices(None, "0,9", runner=r, reexec=False)
    with pytest.raises(mm.MPSConfigError):
        mm.resolve_visible_devices(None, "a,b", runner=r, reexec=False)
    with pytest.raises(mm.MPSConfigError):  # strict under MPS: never change the variable
        mm.resolve_visible_devices(None, "0,1", use_mps=True, runner=r, reexec=False)
    assert os.environ["CUDA_VISIBLE_DEVICES"] == "4,5,6"


def test_daemon_lifecycle_and_env_restore(tmp_path):
    r = FakeRunner()
    m = mm.MPSManager(pipe_dir=str(tmp_path / "pipe"), log_dir=str(tmp_path / "log"), runner=r, register_handlers=False)
    assert m.start() is True and r.daemon and os.environ["NCCL_LAUNCH_MODE"] == "PARALLEL"
    m2 = mm.MPSManager(pipe_dir=str(tmp_path / "pipe"), log_dir=str(tmp_path / "log"), runner=r, register_handlers=False)
    assert m2.start() is False          # re-used, so m2 must not stop it
    m2.stop()
    assert r.daemon
    m.stop()
    assert not r.daemon and "NCCL_LAUNCH_MODE" not in os.environ and "CUDA_MPS_PIPE_DIRECTORY" not in os.environ


def test_stale_pipe_dir_is_cleaned(tmp_path):
    pipe = tmp_path / "pipe"
    pipe.mkdir()
    (pipe / "control").write_text("stale")
    r = FakeRunner()
    m = mm.MPSManager(pipe_dir=str(pipe), log_dir=str(tmp_path / "log"), runner=r, register_handlers=False)
    m.start()
    assert not (pipe / "control").exists()
    m.stop()


def test_file_barrier(tmp_path):
    b = mm.FileBarrier(str(tmp_path), timeout_s=0.3)
    with pytest.raises(TimeoutError):
        b.wait()
    b.signal_abort("daemon failed")
    with pytest.raises(RuntimeError):
        b.wait()
    b.clear()
    b.signal_ready()
    b.wait()


def test_package_imports_without_torch():
    import subprocess
    import sys
    code = "import sys; import aicomp_b200.utils.mps_manager; assert 'torch' not in sys.modules; print('ok')"
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True,
                         cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert out.stdout.strip() == "ok", out.stderr
