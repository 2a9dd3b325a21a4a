"""The C++ host mirror (host/talker_attention_b200.hpp): compiles on CPU, runs on the GPU."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "qingming-qwen3-tts_b200"
BINARY = ROOT / "tests" / "cpp" / "host_mirror_test.bin"


def build_binary(qm):
    qm.build_library()
    from oracle import qm_oracle

    qm_oracle.lib()
    cmd = ["nvcc", "-std=c++17", "-O2", "-I", str(ROOT / "include"), "-I", str(PKG / "host"),
           str(ROOT / "tests" / "cpp" / "host_mirror_test.cpp"), "-o", str(BINARY),
           "-L", str(PKG / "lib"), "-lqm_attention_b200", "-L", str(ROOT / "oracle"), "-lqm_oracle",
           "-Xlinker", f"-rpath={PKG / 'lib'}", "-Xlinker", f"-rpath={ROOT / 'oracle'}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stdout + proc.stderr


def test_host_mirror_compiles_against_the_c_abi(qm):
    build_binary(qm)
    assert BINARY.exists()


@pytest.mark.gpu
def test_host_mirror_prefill_then_decode_matches_oracle(qm):
    if not BINARY.exists():
        build_binary(qm)
    proc = subprocess.run([str(BINARY)], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "HOST_MIRROR_OK" in proc.stdout
