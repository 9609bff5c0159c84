"""Builds and runs the C++ host-side mirror's own tests (tests/cpp/test_host_mirror.cpp): the reference's known
answers replayed through oxidizr_b200/cpp/oxz.hpp over the C ABI, as a compiled client of the library would."""
import os
import subprocess

import pytest

import oxidizr_b200 as ox

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "_build", "test_host_mirror")


def build():
    src = os.path.join(ROOT, "tests", "cpp", "test_host_mirror.cpp")
    hdr = os.path.join(ROOT, "oxidizr_b200", "cpp", "oxz.hpp")
    if os.path.exists(EXE) and os.path.getmtime(EXE) >= max(os.path.getmtime(src), os.path.getmtime(hdr), os.path.getmtime(ox.ffi.LIB_PATH)):
        return
    os.makedirs(os.path.dirname(EXE), exist_ok=True)
    libdir = os.path.dirname(ox.ffi.LIB_PATH)
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    subprocess.run([cxx, "-std=c++17", "-O1", "-Wall", "-o", EXE, src, f"-L{libdir}", "-l:liboxz_dpstep.so",
                    f"-Wl,-rpath,{libdir}", "-pthread"], check=True)


def test_cpp_mirror_replays_the_known_answers_without_a_gpu():
    build()
    out = subprocess.run([EXE], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "all passed" in out.stdout


@pytest.mark.gpu
def test_cpp_mirror_steps_on_the_gpu():
    build()
    out = subprocess.run([EXE, "--gpu"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "all passed" in out.stdout
