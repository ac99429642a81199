"""Compiles and runs tests/host_tables_check.cpp: the integer identities behind the device kernels, checked on the CPU
against the reference's definitions (balanced residue, step-by-step Garner)."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def test_integer_identities(tmp_path):
    exe = str(tmp_path / "host_tables_check")
    subprocess.run(["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-I", os.path.join(ROOT, "ozaki_blackwell_b200", "csrc"),
                    os.path.join(HERE, "host_tables_check.cpp"), "-o", exe], check=True)
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip() == "0 wrong", out.stdout + out.stderr
