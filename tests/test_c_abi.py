"""The drop-in boundary is a C ABI: a plain C99 program (tests/c_abi/metadata_client.c) includes
include/raptor_b200.h, links against the built library and gets the oracle's block tables."""
import os
import shutil
import subprocess

import numpy as np
import pytest

import oracle
from oracle import EncoderConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build_client(tmp_path):
    from raptor_t_b200 import build
    lib = build.build()
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    exe = str(tmp_path / "metadata_client")
    src = os.path.join(ROOT, "tests", "c_abi", "metadata_client.c")
    libdir = os.path.dirname(lib)
    subprocess.check_call([gcc, "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), src,
                           "-o", exe, "-L", libdir, "-lraptor_b200", "-Wl,-rpath," + libdir])
    return exe


def test_header_is_plain_c(tmp_path):
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    src = tmp_path / "only_header.c"
    src.write_text('#include "raptor_b200.h"\nint main(void) { return RT_OK; }\n')
    subprocess.check_call([gcc, "-std=c99", "-Wall", "-Werror", "-pedantic", "-fsyntax-only", "-I",
                           os.path.join(ROOT, "include"), str(src)])


def test_c_client_gets_the_oracle_tables(tmp_path):
    exe = _build_client(tmp_path)
    lens, seed = [1024, 832, 704, 1984], 5
    out = subprocess.run([exe, str(seed)] + [str(n) for n in lens], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    got = {}
    for line in out.stdout.splitlines():
        key, *vals = line.split()
        got[key] = np.array([int(v) for v in vals], dtype=np.int64)
    cfg = EncoderConfig()
    kv_ptr, kv_idx = oracle.build_block_csr(lens, cfg, seed)
    assert got["version"][0] >= 100
    assert np.array_equal(got["prefix"], oracle.seq_block_prefix(lens))
    assert got["visits"][0] == kv_ptr[-1]
    assert np.array_equal(got["kv_ptr"], kv_ptr)
    assert np.array_equal(got["kv_idx"], np.asarray(kv_idx).reshape(-1))
    assert got["bad_status"][0] == 2 and got["bad_message_chars"][0] > 10   # RT_ERR_UNSUPPORTED for 768 tokens
