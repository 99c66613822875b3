"""C++ tests of the shim: its contract against the built library (no GPU needed: every check fails
validation before CUDA is touched), the persistent kernels' work distribution (plain arithmetic
shared by host and device), and -- on a GPU -- the join rules and the plan cache on device memory."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
CUDA_INCLUDE = Path("/usr/local/cuda/include")


@pytest.mark.skipif(shutil.which("g++") is None or not CUDA_INCLUDE.exists(), reason="needs g++ and the CUDA headers")
def test_shim_contract(tmp_path):
    from gewell_b200 import _lib
    assert _lib.LIBRARY_PATH.exists(), "build the library first: python -m gewell_b200.build"
    exe = tmp_path / "shim_contract"
    subprocess.run(["g++", "-std=c++17", "-I", str(ROOT / "include"), "-I", str(CUDA_INCLUDE),
                    str(ROOT / "tests" / "cpp" / "shim_contract.cpp"), "-o", str(exe),
                    str(_lib.LIBRARY_PATH), f"-Wl,-rpath,{_lib.LIBRARY_PATH.parent}",
                    "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,/usr/local/cuda/lib64"], check=True)
    done = subprocess.run([str(exe)], capture_output=True, text=True)
    assert done.returncode == 0, done.stdout + done.stderr
    assert "PASS" in done.stdout


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_work_distribution_covers_every_item_once(tmp_path):
    exe = tmp_path / "work_walk_test"
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", str(ROOT / "gewell_b200" / "csrc"),
                    str(ROOT / "tests" / "cpp" / "work_walk_test.cpp"), "-o", str(exe)], check=True)
    done = subprocess.run([str(exe)], capture_output=True, text=True)
    assert done.returncode == 0, done.stdout + done.stderr
    assert "PASS" in done.stdout


def _build(tmp_path, source: str) -> Path:
    from gewell_b200 import _lib
    assert _lib.LIBRARY_PATH.exists(), "build the library first: python -m gewell_b200.build"
    exe = tmp_path / Path(source).stem
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", str(ROOT / "include"), "-I", str(CUDA_INCLUDE),
                    str(ROOT / "tests" / "cpp" / source), "-o", str(exe),
                    str(_lib.LIBRARY_PATH), f"-Wl,-rpath,{_lib.LIBRARY_PATH.parent}",
                    "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,/usr/local/cuda/lib64"], check=True)
    return exe


@pytest.mark.skipif(shutil.which("g++") is None or not CUDA_INCLUDE.exists(), reason="needs g++ and the CUDA headers")
def test_shim_device_program_compiles(tmp_path):
    """The device test program builds against the shim (its run needs a GPU: see below)."""
    assert _build(tmp_path, "shim_device.cpp").exists()


@pytest.mark.gpu
def test_shim_join_rules_on_device(tmp_path):
    """Joined gate/up == separate GEMMs bit for bit (NVFP4 and FP8 with per-channel scales), join
    rejections, fused GeGLU input == GeGLU then projection, plan cache with one shared scratch."""
    exe = _build(tmp_path, "shim_device.cpp")
    done = subprocess.run([str(exe)], capture_output=True, text=True)
    assert done.returncode == 0, done.stdout + done.stderr
    assert "PASS" in done.stdout
