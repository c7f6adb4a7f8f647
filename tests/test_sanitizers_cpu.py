"""The host runtime under ThreadSanitizer and AddressSanitizer: the library is rebuilt with the sanitizer, the
native unit tests and the forked 3-rank test (negotiated collectives, fused tensors, sparse and dense parameter
servers over the TCP meshes) are linked against it and must finish without a report."""
import os
import subprocess

import pytest


@pytest.mark.parametrize("sanitizer", ["thread", "address"])
def test_native_tests_are_clean_under_the_sanitizer(sanitizer):
    from tips_b200 import build
    probe = subprocess.run([build.CXX, f"-fsanitize={sanitizer}", "-x", "c++", "-", "-o", os.devnull],
                           input="int main(){return 0;}", capture_output=True, text=True)
    if probe.returncode != 0:
        pytest.skip(f"the toolchain has no {sanitizer} sanitizer runtime")
    exes = build.build_native_tests(sanitize=sanitizer)
    assert {e.name for e in exes} >= {f"core_test_{sanitizer}", f"ranks_test_{sanitizer}"}
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66 second_deadlock_stack=1",
               ASAN_OPTIONS="detect_leaks=1 exitcode=67")
    for exe in exes:
        r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600, env=env)
        report = [l for l in (r.stdout + r.stderr).splitlines() if "Sanitizer" in l]
        assert r.returncode == 0 and not report, f"{exe.name}: rc {r.returncode}\n" + "\n".join(report[:20]) + r.stderr[-2000:]


def test_message_benchmark_runs():
    import ctypes
    from tips_b200 import _lib
    lib = _lib.core()
    lib.tips_bench_messages.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
    out = (ctypes.c_double * 4)()
    assert lib.tips_bench_messages(1000, out) == 0
    assert all(0 < v < 1e6 for v in out)   # nanoseconds per message
