"""Host-side native tests under AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer.

The GPU pool offers no memory checker, so the device code is guarded by guard bands, bounded waits and the per-tile
staging check; the host side of the library (proxy threads, bootstraps, verbs providers, shared-memory regions, the
CPU ring) is checked here: the programs are rebuilt with the sanitizer (no shared library, no device code) and must
run clean."""
import os
import subprocess

import pytest


@pytest.mark.parametrize("kind", ["address", "thread"])
def test_host_programs_run_clean_under_the_sanitizer(kind, native_build):
    if native_build.sanitizer_compiler(kind) is None:
        pytest.skip(f"no compiler here links with -fsanitize={kind}")
    programs = native_build.build_sanitized(kind)
    assert len(programs) >= 5
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1",
               TSAN_OPTIONS="halt_on_error=0:exitcode=66")
    for exe in programs:
        p = subprocess.run([str(exe)], capture_output=True, text=True, timeout=900, env=env)
        text = p.stdout + p.stderr
        assert p.returncode == 0 and "Sanitizer" not in text, f"{exe.name}:\n{text[-4000:]}"
