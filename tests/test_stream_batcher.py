"""host/stream_batcher.hpp: the page allocator and request batcher.  Its logic is checked on the CPU by a C++
program (scripted answers + a seeded random simulation with invariants); on the GPU a second program lets streams
join and leave between decode steps and compares every stream's context with the oracle run on that stream alone."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "qingming-qwen3-tts_b200"
CPU_BINARY = ROOT / "tests" / "cpp" / "stream_batcher_test.bin"
GPU_BINARY = ROOT / "tests" / "cpp" / "stream_batcher_gpu_test.bin"


def build_gpu_binary(qm):
    qm.build_library()
    from oracle import qm_oracle

    qm_oracle.lib()
    cmd = ["nvcc", "-std=c++17", "-O2", "-I", str(ROOT / "include"), "-I", str(PKG / "host"),
           str(ROOT / "tests" / "cpp" / "stream_batcher_gpu_test.cpp"), "-o", str(GPU_BINARY),
           "-L", str(PKG / "lib"), "-lqm_attention_b200", "-L", str(ROOT / "oracle"), "-lqm_oracle",
           "-Xlinker", f"-rpath={PKG / 'lib'}", "-Xlinker", f"-rpath={ROOT / 'oracle'}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stdout + proc.stderr


def test_batcher_logic_on_cpu():
    cmd = ["g++", "-std=c++17", "-O2", "-Wall", "-Werror", "-I", str(PKG / "host"),
           str(ROOT / "tests" / "cpp" / "stream_batcher_test.cpp"), "-o", str(CPU_BINARY)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    proc = subprocess.run([str(CPU_BINARY)], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "STREAM_BATCHER_OK" in proc.stdout


def test_batcher_gpu_program_compiles_against_the_c_abi(qm):
    build_gpu_binary(qm)
    assert GPU_BINARY.exists()


@pytest.mark.gpu
def test_streams_join_and_leave_between_decode_steps(qm):
    if not GPU_BINARY.exists():
        build_gpu_binary(qm)
    proc = subprocess.run([str(GPU_BINARY)], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "STREAM_BATCHER_GPU_OK" in proc.stdout
