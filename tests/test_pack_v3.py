"""The "tokspur-pack-v3" container reader of the C++ host layer, on the CPU: runs native/tests/test_pack_v3_cpu.cpp, which writes
a small layer in the reference's pack layouts with the test-side writer, reads it back field by field, checks the refusals of
damaged files and - where the reference's CPU sources were compiled (oracle/_ref) - compares the directory with what the
reference's own GGUF parser makes of the same bytes."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NATIVE = os.path.join(ROOT, "tokspur-public_b200", "native")
BIN = os.path.join(NATIVE, "tests", "test_pack_v3_cpu")


def test_pack_v3_reader_cpu_suite():
    if not os.path.exists(os.path.join(ROOT, "oracle", "liboracle.so")):
        subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle")], check=True)
    subprocess.run(["make", "-s", "-C", NATIVE, BIN], check=True)
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "pack v3 reader checks passed" in r.stdout
    if os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libtokspur_ref.so")):
        assert "reference GGUF parser agrees" in r.stdout
