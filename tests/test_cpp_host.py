"""The C++ host layer (include/b200nn.hpp: the reference's `nn` names as RAII classes over the C ABI):
it compiles with the system C++ compiler, links against the library, refuses to run without a CUDA
device, and on a GPU its checks against plain host arithmetic pass (tests/cpp/host_mirror.cpp)."""
import os
import subprocess

import pytest

import b200nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "host_mirror.cpp")
OUT_DIR = os.path.join(ROOT, "tests", "cpp", "_build")
EXE = os.path.join(OUT_DIR, "host_mirror")


def _build():
    b200nn.load_library()  # builds libb200nn.so when it is missing
    lib_dir = os.path.dirname(b200nn.LIB_PATH)
    deps = [SRC, os.path.join(ROOT, "include", "b200nn.hpp"), os.path.join(ROOT, "include", "b200nn.h")]
    if os.path.exists(EXE) and all(os.path.getmtime(EXE) >= os.path.getmtime(d) for d in deps):
        return
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-I", os.path.join(ROOT, "include"), SRC,
           "-L", lib_dir, "-lb200nn", "-Wl,-rpath,$ORIGIN/" + os.path.relpath(lib_dir, OUT_DIR), "-o", EXE]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_cpp_host_layer_compiles_and_fails_loudly_without_a_device():
    import torch
    _build()
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present: the run is covered by the gpu test")
    r = subprocess.run([EXE], capture_output=True, text=True, timeout=120)
    assert r.returncode == 3 and r.stdout.startswith("NO_DEVICE: Cuda"), (r.returncode, r.stdout, r.stderr)


@pytest.mark.gpu
def test_cpp_host_layer_on_the_gpu():
    _build()
    r = subprocess.run([EXE], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().splitlines()[-1].startswith("OK "), (r.returncode, r.stdout, r.stderr)
