"""Host-only checks of the C ABI: the library loads, exports every symbol the header
declares, and follows the reference wrapper's error convention for calls that need no GPU
(src/k4/ter_k4.cpp:22-72, pinned there by tests/test_ter_k4.cpp:21-23)."""
import ctypes as C
import os
import re

import pytest

from ter_b200 import api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            txt = open(os.path.join(ROOT, "include", fn)).read()
            txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
            names |= set(re.findall(r"\b(ter_b200_[a-z0-9_]+)\s*\(", txt))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    L = api.load()
    syms = declared_symbols()
    assert len(syms) >= 20
    for s in syms:
        assert hasattr(L, s), f"{s} declared in include/ but not exported"
        assert s in api.SIGNATURES, f"{s} has no ctypes signature in ter_b200/api.py"


def test_null_handle_conventions():
    L = api.load()
    assert L.ter_b200_call(None, b"tk_matmul_b_9t", None, 0) == api.E_NULL
    assert L.ter_b200_install_kernel(None, b"w", b"\0" * 64, 16) == api.E_NULL
    assert L.ter_b200_install_weight(None, b"w", None, 0, 16, 4, 1.0) == api.E_NULL
    assert L.ter_b200_gemv(None, b"w", None, None, None, None) == api.E_NULL
    assert L.ter_b200_gemm(None, b"w", None, None, 1, None, None) == api.E_NULL
    assert L.ter_b200_sync(None, None) == api.E_NULL
    assert L.ter_b200_device_status(None) == api.E_NULL
    # void functions silently ignore NULL (src/k4/ter_k4.cpp:61-72)
    L.ter_b200_destroy(None)
    L.ter_b200_reset_counters(None)
    c = api.OpCounts(1, 2, 3, 4, 5)
    L.ter_b200_op_counts(None, C.byref(c))
    assert c.tvmac == 2
    assert L.ter_b200_launch_count(None) == 0


def test_strerror_covers_all_codes():
    L = api.load()
    seen = set()
    for code in range(0, -13, -1):
        s = L.ter_b200_strerror(code).decode()
        assert s and s != "unknown error code"
        seen.add(s)
    assert len(seen) == 13
    assert L.ter_b200_strerror(-99).decode() == "unknown error code"


def test_create_without_gpu_returns_null():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = api.load()
    assert L.ter_b200_create(0) is None
    with pytest.raises(RuntimeError):
        api.TerB200(0)


def test_packed_model_file_header_round_trip(tmp_path):
    """The writer and the library's header reader agree on the reference's 64-byte header
    (tools/convert_llama_to_packed.py:13-24); foreign and short files are return codes."""
    import numpy as np
    from ter_b200 import modelfile, synth
    cfg = dict(arch=1, H=128, F=256, L=1, V=512, Nh=2, Nkv=1, Hd=64, Smax=48, eps=1e-5, rope_theta=500000.0)
    path = str(tmp_path / "tiny_tert.bin")
    modelfile.write_packed_model(path, cfg, synth.model_weights(cfg, 5))
    Hkv = cfg["Nkv"] * cfg["Hd"]
    per_layer = 4 * (3 * cfg["H"] + cfg["F"]) + 7 * 4 + (2 * cfg["H"] * cfg["H"] + 2 * cfg["H"] * Hkv + 3 * cfg["H"] * cfg["F"]) // 4
    assert os.path.getsize(path) == 64 + 2 * cfg["V"] * cfg["H"] + 4 * cfg["H"] + cfg["L"] * per_layer
    got = api.model_file_info(path)
    for k in ("arch", "H", "F", "L", "V", "Nh", "Nkv", "Hd", "Smax"):
        assert got[k] == cfg[k], k
    assert got["eps"] == np.float32(cfg["eps"]) and got["rope_theta"] == cfg["rope_theta"]
    assert modelfile.read_header(path)["arch"] == 1
    L = api.load()
    c = api.ModelCfg()
    assert L.ter_b200_model_file_info(None, C.byref(c)) == api.E_NULL
    assert L.ter_b200_model_file_info(str(tmp_path / "missing.bin").encode(), C.byref(c)) == api.E_IO
    bad = tmp_path / "bad.bin"
    bad.write_bytes(b"GGUF" + b"\0" * 100)
    assert L.ter_b200_model_file_info(str(bad).encode(), C.byref(c)) == api.E_IO
    short = tmp_path / "short.bin"
    short.write_bytes(open(path, "rb").read(40))
    assert L.ter_b200_model_file_info(str(short).encode(), C.byref(c)) == api.E_IO
    assert L.ter_b200_model_load_file(None, path.encode(), 0, 1, None) == api.E_NULL
