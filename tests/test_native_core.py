"""Native L0/L3 unit tests (C++ executable) and library loading."""
import subprocess


def test_native_core_executable():
    from tips_b200 import build
    exes = build.build_native_tests()
    assert exes
    for exe in exes:
        r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, r.stdout + r.stderr


def test_c_api_lifecycle_single_rank(monkeypatch):
    import socket
    from tips_b200 import _lib
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    lib = _lib.core()
    assert lib.tips_is_initialized() == 0 and lib.tips_rank() == -1
    assert lib.tips_init_ex(0, 1, b"127.0.0.1", port) == 0
    assert lib.tips_is_initialized() == 1 and lib.tips_is_initialize() == 1
    assert lib.tips_rank() == 0 and lib.tips_size() == 1 and lib.tips_local_rank() == 0
    assert lib.tips_barrier() == 0
    assert lib.tips_shutdown() == 0
    assert lib.tips_is_initialized() == 0
    # a second life in the same process
    assert lib.tips_init_ex(0, 1, b"127.0.0.1", port) == 0
    assert lib.tips_shutdown() == 0
