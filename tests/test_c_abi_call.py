"""Builds tests/c_abi_call.c against include/arattn.h and runs it: a C program that calls the six
ops.mojo mirrors in the reference trainer's order with the reference's argument order, as the Mojo
binding (mojo/attn_ffi.mojo) would.  The CPU test only compiles and links it; the GPU test runs it
on seeded inputs and compares its output file with the oracle."""
import os
import subprocess

import numpy as np
import pytest

import autoresearch_b200 as ab
from oracle import oracle as orc
from tests.parity_util import assert_parity

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def build(tmp_path):
    exe = tmp_path / "c_abi_call"
    libdir = os.path.dirname(ab.lib_path())
    subprocess.check_call([
        "gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-O1",
        "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"),
        os.path.join(ROOT, "tests", "c_abi_call.c"), "-o", str(exe),
        "-L", libdir, "-larattn", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
        f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{os.path.join(CUDA, 'lib64')}"])
    return exe


def test_c_caller_compiles_and_links_against_the_header(tmp_path):
    exe = build(tmp_path)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 1 and "usage" in r.stderr


@pytest.mark.gpu
def test_c_caller_matches_the_oracle(cuda_device, tmp_path):
    exe = build(tmp_path)
    B, T, H, W = 2, 300, 3, 100
    q, k, v, do = orc.make_inputs(B, T, H, 128, seed=17, bf16=True)
    cos, sin = orc.rope_table(T, 128)
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(fin, "wb") as f:
        for a in (q, k, v, do, cos, sin):
            f.write(np.ascontiguousarray(a, np.float32).tobytes())
    r = subprocess.run([str(exe), str(fin), str(fout), str(B), str(T), str(H), str(W)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    raw = np.fromfile(fout, np.float32)
    n, rows = B * T * H * 128, B * T * H
    sizes = [("o", n, (B, T, H, 128)), ("lse", rows, (B, T, H)), ("d", rows, (B, T, H)),
             ("dq", n, (B, T, H, 128)), ("dk", n, (B, T, H, 128)), ("dv", n, (B, T, H, 128))]
    got, off = {}, 0
    for name, cnt, shape in sizes:
        got[name] = raw[off:off + cnt].reshape(shape)
        off += cnt
    assert off == raw.size
    # The mirrors round the rotated q, k to bf16 when they stage them; the oracle gets the same
    # inputs and rotates in fp32, so this comparison also covers that rounding.
    want = orc.attention_path(q, k, v, do, W, rope=(cos, sin))
    assert_parity({n: orc.parity(got[n], want[n]) for n in ("o", "lse", "dq", "dk", "dv")}, what="C caller")
