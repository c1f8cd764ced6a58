"""Environment diagnostics (the reference's tests/python/test_env.py shape)."""

import subprocess
import sys
import types

import swage_b200
from swage_b200 import env


def test_version_present():
    assert swage_b200.__version__
    assert swage_b200.__version__[0].isdigit()


def test_report_keys():
    result = env.report()
    for key in ("swage_b200", "python", "platform", "torch",
                "torch_cuda_build", "cuda_driver", "cuda", "gpu", "library",
                "backends"):
        assert key in result


def test_report_separates_torch_build_from_cuda_driver(monkeypatch):
    torch = types.SimpleNamespace(
        __version__="2.11.0",
        version=types.SimpleNamespace(cuda="12.8"),
        cuda=types.SimpleNamespace(
            is_available=lambda: True,
            get_device_capability=lambda: (10, 0),
            get_device_name=lambda: "NVIDIA B200",
        ),
    )
    monkeypatch.setattr(env.importlib.util, "find_spec", lambda _name: object())
    monkeypatch.setitem(sys.modules, "torch", torch)
    monkeypatch.setattr(env, "driver_version", lambda: "13.0")
    result = env.report()
    assert result["torch_cuda_build"] == "12.8"
    assert result["cuda_driver"] == "13.0"
    assert result["gpu"] == {"name": "NVIDIA B200",
                             "compute_capability": "10.0"}


def test_backends_line_is_truthful(monkeypatch, native_library):
    # no device: never "available", whatever is built
    torch = types.SimpleNamespace(
        __version__="2.11.0", version=types.SimpleNamespace(cuda="12.8"),
        cuda=types.SimpleNamespace(is_available=lambda: False))
    monkeypatch.setattr(env.importlib.util, "find_spec", lambda _name: object())
    monkeypatch.setitem(sys.modules, "torch", torch)
    result = env.report()
    assert result["backends"]["cuda_sm100a"].startswith("unavailable")
    assert "no CPU fallback" in result["backends"]["cpu"]
    # a device of another architecture cannot run sm_100a code
    torch.cuda = types.SimpleNamespace(
        is_available=lambda: True, get_device_capability=lambda: (9, 0),
        get_device_name=lambda: "H100")
    monkeypatch.setattr(env, "driver_version", lambda: "12.9")
    assert "sm_100a code only" in env.report()["backends"]["cuda_sm100a"]
    torch.cuda.get_device_capability = lambda: (10, 0)
    assert env.report()["backends"]["cuda_sm100a"].startswith("available")


def test_missing_library_is_reported_not_raised(monkeypatch, tmp_path):
    from swage_b200 import _native

    monkeypatch.setattr(_native, "LIBRARY_PATH", tmp_path / "absent.so")
    result = env.report()
    assert "not built" in result["library"]
    assert result["backends"]["cuda_sm100a"].startswith("unavailable")


def test_module_entrypoint():
    proc = subprocess.run([sys.executable, "-m", "swage_b200.env"],
                          capture_output=True, text=True, check=True)
    assert "swage_b200:" in proc.stdout
    assert "python:" in proc.stdout
    assert "backends:" in proc.stdout
