"""The native host core (pages, block tables, step assembly, scheduler decisions) built with the address and
undefined-behaviour sanitizers and driven by the cache, scheduler and step-assembly tests: random orders of
requests, pools that run out, refused batches.  The reference builds without sanitizers and relies on a
single-threaded engine (src/locus/engine/engine.hpp:79-81); this is the check that its counterpart here
touches no memory it does not own."""
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _checked_compiler():
    """(compiler, libasan, libubsan) of the first C++ compiler that ships both sanitizer runtimes."""
    for cand in (os.environ.get("CXX"), "g++", "c++", "/usr/bin/g++", "clang++"):
        cxx = shutil.which(cand) if cand else None
        if cxx is None:
            continue
        libs = []
        for name in ("libasan.so", "libubsan.so"):
            path = subprocess.run([cxx, f"-print-file-name={name}"], capture_output=True, text=True).stdout.strip()
            if os.path.isabs(path) and os.path.exists(path):
                libs.append(os.path.realpath(path))
        if len(libs) == 2:
            return cxx, libs[0], libs[1]
    return None


def test_cache_and_scheduler_tests_under_sanitizers(tmp_path):
    found = _checked_compiler()
    if found is None:
        pytest.skip("no C++ compiler with the sanitizer runtimes")
    cxx, asan, ubsan = found
    env = dict(os.environ)
    env.update({
        "CXX": cxx,
        "LOCUS_HOST_FLAGS": "-fsanitize=address,undefined -fno-omit-frame-pointer -g",
        "LOCUS_BUILD_DIR": str(tmp_path),            # the checked library never lands beside the regular one
        "LD_PRELOAD": f"{asan}:{ubsan}",              # the interpreter itself is not instrumented
        "ASAN_OPTIONS": "detect_leaks=0:halt_on_error=1:abort_on_error=0",
        "UBSAN_OPTIONS": "halt_on_error=1:print_stacktrace=1",
    })
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-m", "not gpu", "-p", "no:cacheprovider",
           os.path.join(ROOT, "tests", "test_cache.py"), os.path.join(ROOT, "tests", "test_scheduler.py"),
           os.path.join(ROOT, "tests", "test_engine_host.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    out = r.stdout + r.stderr
    assert "AddressSanitizer" not in out and "runtime error:" not in out, out[-4000:]
    assert r.returncode == 0, out[-4000:]
    built = [f for f in os.listdir(tmp_path) if f.startswith("libhost_core-") and f.endswith(".so")]
    assert built, "the checked library was not built"
