"""The native cache manager under AddressSanitizer and UndefinedBehaviorSanitizer: a C++ driver (host_stress.cpp)
opens, reserves, describes, commits, cancels and closes at random, with an audit after every operation."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def test_random_operations_under_sanitizers(tmp_path):
    exe = str(tmp_path / "host_stress")
    compilers = [c for c in dict.fromkeys(shutil.which(n) for n in (os.environ.get("CXX"), "g++", "c++", "clang++") if n) if c]
    if not compilers:
        pytest.skip("no C++ compiler")
    errors = []
    for cxx in compilers:                    # (a compiler may come without the sanitizers' runtime libraries)
        cmd = [cxx, "-O1", "-g", "-std=c++17", "-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-o", exe,
               os.path.join(HERE, "host_stress.cpp"), os.path.join(ROOT, "xyntetik_runner_b200", "csrc", "host", "page_cache.cpp")]
        built = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
        if built.returncode == 0:
            break
        errors.append(f"{cxx}: {built.stderr[-300:]}")
        assert "asan" in built.stderr or "ubsan" in built.stderr or "sanitize" in built.stderr, built.stderr
    else:
        pytest.skip("no compiler here has the sanitizer libraries: " + " | ".join(errors))
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and run.stdout.strip() == "ok", run.stdout + run.stderr
