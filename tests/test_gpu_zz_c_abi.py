"""The C ABI is usable from plain C: examples/c_abi_axpy.c compiles as C99 against
include/cnb200.h with warnings on, links against the library, builds a DAG blob by hand that is
byte-identical to what the Python writer produces for the same expression, and -- on a machine
without a GPU -- fails loudly at context creation instead of computing anything."""
import shutil
import subprocess
from pathlib import Path

import pytest

from charmnumeric_b200 import wire
from charmnumeric_b200._lib import LIB_PATH

ROOT = Path(__file__).resolve().parent.parent
CC = shutil.which("gcc") or shutil.which("cc")


@pytest.fixture(scope="module")
def binary(tmp_path_factory):
    if CC is None:
        pytest.skip("no C compiler")
    out = tmp_path_factory.mktemp("c_abi") / "c_abi_axpy"
    libdir = str(Path(LIB_PATH).parent)
    res = subprocess.run([CC, "-std=c99", "-Wall", "-Wextra", "-Werror", "-I", str(ROOT / "include"),
                          str(ROOT / "examples" / "c_abi_axpy.c"), "-L", libdir, "-lcnb200",
                          f"-Wl,-rpath,{libdir}", "-o", str(out)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return out


def test_hand_built_blob_is_what_the_python_writer_builds(binary, tmp_path):
    dump = tmp_path / "blob.bin"
    res = subprocess.run([str(binary), "--check", str(dump)], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    n = 32
    roots = [
        wire.Ast(10, wire.OP_ADD, is_temp=True, shape=(n,),
                 operands=[(wire.leaf(1, (n,)), None), (wire.leaf(2, (n,)), None)]),
        wire.Ast(11, wire.OP_ADD, is_temp=True, shape=(n,),
                 operands=[(wire.Ref(10), None), (wire.scalar(3.0), None)]),
        wire.Ast(3, wire.OP_MUL, shape=(n,), operands=[(wire.scalar(2.0), None), (wire.Ref(11), None)]),
    ]
    expected = wire.dag_blob([wire.Node(0, roots, identifier=1)], [], 1)
    assert dump.read_bytes() == expected


def test_without_a_gpu_the_program_fails_loudly(binary):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the GPU run is covered by test_gpu_c_abi_example")
    res = subprocess.run([str(binary)], capture_output=True, text=True)
    assert res.returncode == 2
    assert "no CUDA device" in res.stderr


@pytest.mark.gpu
def test_gpu_c_abi_example(binary):
    res = subprocess.run([str(binary)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "= 8 on all 32 elements" in res.stdout
