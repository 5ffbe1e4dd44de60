"""Builds and runs the C++ test of the host mirror (config validation transcribed from the reference's tests)."""
import os
import subprocess

from singe_b200 import kernel_sys as ks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_host_mirror_validation(tmp_path):
    if not os.path.exists(ks.LIB_PATH):
        from singe_b200 import build

        build.build()
    binary = tmp_path / "test_host_mirror"
    library_dir = os.path.dirname(ks.LIB_PATH)
    subprocess.run(["/usr/bin/g++", "-std=c++17", "-O1", "-Wall", os.path.join(ROOT, "tests", "host", "test_host_mirror.cpp"),
                    "-o", str(binary), f"-L{library_dir}", "-lsinge_kernel_sys", f"-Wl,-rpath,{library_dir}",
                    "-L/usr/local/cuda/lib64", "-Wl,-rpath,/usr/local/cuda/lib64"], check=True)
    result = subprocess.run([str(binary)], capture_output=True, text=True)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "host mirror ok" in result.stdout
