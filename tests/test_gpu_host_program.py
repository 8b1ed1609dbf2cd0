"""A host program without Python: tests/cpp/host_program.cpp is compiled against
include/b200mlir_capi.h, linked with the shared library and run — one forked process per GPU.
It runs `matmul` and the tensor-parallel MLP block (the library's own NCCL communicator, created
from an id that rank 0 hands the others through a pipe; ncclAllReduce inside
`mlp_block_tp_float16`) and, on two ranks, a host-buffer `matmul` whose A every rank holds (row
slabs uploaded per rank and exchanged between the GPUs), and checks all three against CPU loops
of its own."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def program(hm, tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("cpp") / "host_program")
    libdir = os.path.dirname(hm.LIB_PATH)
    cmd = ["g++", "-std=c++17", "-O2", f"-I{os.path.join(ROOT, 'include')}", os.path.join(ROOT, "tests", "cpp", "host_program.cpp"),
           "-o", exe, f"-L{libdir}", "-lb200mlir", f"-Wl,-rpath,{libdir}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def run(exe, world):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")   # a test in which a rank may fail: no multicast bindings
    r = subprocess.run([exe, str(world)], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all ranks ok" in r.stdout
    return r.stdout


def test_single_rank(program, cuda):
    out = run(program, 1)
    assert "matmul 384x512x320" in out and "rank 0 of 1: mlp block (chunks 2)" in out


def test_two_ranks_nccl_all_reduce_in_cpp(program, cuda):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = run(program, 2)
    assert "rank 1 of 2: mlp block (chunks 1)" in out and "rank 0 of 2: mlp block (chunks 2)" in out
    assert "rank 0 of 2: host-buffer matmul, replicated A, 8 x 4 panels" in out
    assert "rank 1 of 2: host-buffer matmul, replicated A, 8 x 4 panels" in out
