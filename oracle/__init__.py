"""TEST INFRASTRUCTURE, NOT PRODUCT CODE.

ctypes bindings to the two CPU checkers:

* ``libter_oracle.so`` - the plain-C restatement (``ter_oracle.c``).
* ``_ref/libter_ref.so`` - the unmodified reference CPU code behind a thin
  C driver (``ref_driver.cpp``); present only where it was built from the
  reference checkout (or carried along as a prebuilt file).

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline
legs import this package.  Nothing under ``ter_b200/`` does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "libter_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libter_ref.so")

ARCH_LLAMA, ARCH_BITNET = 0, 1
WQ, WK, WV, WO, WGATE, WUP, WDOWN = range(7)
ATTN_NORM, FFN_NORM, ATTN_SUB_NORM, FFN_SUB_NORM = range(4)
MAT_NAMES = ["q", "k", "v", "o", "gate", "up", "down"]


def build(ref: str | None = None) -> None:
    """Compile the C restatement, and the reference driver and programs when a reference
    checkout is given (argument, or TER_REFERENCE in the environment)."""
    ref = ref if ref is not None else os.environ.get("TER_REFERENCE", "")
    subprocess.run(["make", "-s", "-C", _HERE, "all", f"REF={ref}"], check=True)


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


class Cfg(C.Structure):
    _fields_ = [("arch", C.c_int), ("H", C.c_int), ("F", C.c_int), ("L", C.c_int),
                ("V", C.c_int), ("Nh", C.c_int), ("Nkv", C.c_int), ("Hd", C.c_int),
                ("Smax", C.c_int), ("eps", C.c_float), ("rope_theta", C.c_double),
                ("lm_head_packed", C.c_int), ("kv_f32", C.c_int), ("np_quant", C.c_int)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build()
        L = C.CDLL(ORACLE_SO)
        L.orc_tvmac.restype = C.c_uint64
        L.orc_quantize_trit.restype = C.c_float
        L.orc_expf.restype = C.c_float
        L.orc_expf.argtypes = [C.c_float]
        L.orc_model_create.restype = C.c_void_p
        L.orc_state_create.restype = C.c_void_p
        L.orc_model_create.argtypes = [C.POINTER(Cfg)]
        L.orc_model_destroy.argtypes = [C.c_void_p]
        L.orc_model_set_matrix.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_float]
        L.orc_model_set_vector.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.orc_model_set_embd.argtypes = [C.c_void_p, C.c_void_p]
        L.orc_model_set_threads.argtypes = [C.c_void_p, C.c_int]
        L.orc_state_create.argtypes = [C.c_void_p, C.c_int]
        L.orc_state_destroy.argtypes = [C.c_void_p]
        L.orc_forward_token.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                        C.c_void_p, C.c_void_p]
        L.orc_state_layer_hidden.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        _lib = L
    return _lib


# ---------------------------------------------------------------- packing
def pack_v11(trits: np.ndarray) -> np.ndarray:
    """trits int8 [K][N] in {-1,0,1} -> bytes [N/4][K]."""
    K, N = trits.shape
    t = np.ascontiguousarray(trits, dtype=np.int8)
    out = np.empty((N // 4, K), dtype=np.uint8)
    lib().orc_pack_v11(_p(t, C.c_int8), K, N, _p(out, C.c_uint8))
    return out


def pack_rowmajor(trits: np.ndarray) -> np.ndarray:
    K, N = trits.shape
    t = np.ascontiguousarray(trits, dtype=np.int8)
    out = np.empty((K, N // 4), dtype=np.uint8)
    lib().orc_pack_rowmajor(_p(t, C.c_int8), K, N, _p(out, C.c_uint8))
    return out


def unpack_v11(packed: np.ndarray, K: int, N: int) -> np.ndarray:
    p = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty((K, N), dtype=np.int8)
    lib().orc_unpack_v11(_p(p, C.c_uint8), K, N, _p(out, C.c_int8))
    return out


def unpack_rowmajor(packed: np.ndarray, K: int, N: int) -> np.ndarray:
    p = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty((K, N), dtype=np.int8)
    lib().orc_unpack_rowmajor(_p(p, C.c_uint8), K, N, _p(out, C.c_int8))
    return out


# ------------------------------------------------------------------ GEMV
def mm_row_acc(X: np.ndarray, W: np.ndarray) -> np.ndarray:
    """int32 X[K], int32 W[K][N] -> int64 accumulators[N]."""
    K, N = W.shape
    X = np.ascontiguousarray(X, dtype=np.int32)
    W = np.ascontiguousarray(W, dtype=np.int32)
    acc = np.empty(N, dtype=np.int64)
    lib().orc_mm_row_acc(_p(X, C.c_int32), _p(W, C.c_int32), K, N, _p(acc, C.c_int64))
    return acc


def mm_row(X, x_scale, W, w_scale) -> np.ndarray:
    K, N = W.shape
    X = np.ascontiguousarray(X, dtype=np.int32)
    W = np.ascontiguousarray(W, dtype=np.int32)
    out = np.empty(N, dtype=np.float32)
    lib().orc_mm_row(_p(X, C.c_int32), C.c_float(x_scale), _p(W, C.c_int32), C.c_float(w_scale),
                     K, N, _p(out, C.c_float))
    return out


def tvmac(K: int, N: int) -> int:
    return int(lib().orc_tvmac(K, N))


def gemv_packed_acc(x: np.ndarray, Wcol: np.ndarray, K: int, N: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.int8)
    Wcol = np.ascontiguousarray(Wcol, dtype=np.uint8)
    acc = np.empty(N, dtype=np.int32)
    lib().orc_gemv_packed_v11_acc(_p(x, C.c_int8), _p(Wcol, C.c_uint8), K, N, _p(acc, C.c_int32))
    return acc


def gemv_acc_fast(x: np.ndarray, trits: np.ndarray) -> np.ndarray:
    """Exact int32 dot products through numpy int64 matmul (large shapes)."""
    return (x.astype(np.int64) @ trits.astype(np.int64)).astype(np.int32)


def gemv_epilogue(acc: np.ndarray, x_scale, w_scale) -> np.ndarray:
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    out = np.empty(acc.shape[0], dtype=np.float32)
    lib().orc_gemv_epilogue(_p(acc, C.c_int32), acc.shape[0], C.c_float(x_scale), C.c_float(w_scale),
                            _p(out, C.c_float))
    return out


def gemm_packed(X: np.ndarray, x_scales: np.ndarray, Wcol: np.ndarray, w_scale, K: int, N: int):
    X = np.ascontiguousarray(X, dtype=np.int8)
    M = X.shape[0]
    xs = np.ascontiguousarray(x_scales, dtype=np.float32)
    Wcol = np.ascontiguousarray(Wcol, dtype=np.uint8)
    acc = np.empty((M, N), dtype=np.int32)
    out = np.empty((M, N), dtype=np.float32)
    lib().orc_gemm_packed_v11(_p(X, C.c_int8), _p(xs, C.c_float), M, _p(Wcol, C.c_uint8),
                              C.c_float(w_scale), K, N, _p(acc, C.c_int32), _p(out, C.c_float))
    return acc, out


# ------------------------------------------------------------- quantisers
def quantize_trit(x: np.ndarray, n_trits: int = 9):
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.empty(x.shape[0], dtype=np.int32)
    s = lib().orc_quantize_trit(_p(x, C.c_float), x.shape[0], n_trits, _p(q, C.c_int32))
    return q, float(s)


def quant_int8(x: np.ndarray):
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.empty(x.shape[0], dtype=np.int8)
    s = C.c_float()
    lib().orc_quant_int8(_p(x, C.c_float), x.shape[0], _p(q, C.c_int8), C.byref(s))
    return q, np.float32(s.value)


def rmsnorm(x, gamma, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    g = np.ascontiguousarray(gamma, dtype=np.float32)
    y = np.empty_like(x)
    lib().orc_rmsnorm(_p(x, C.c_float), _p(g, C.c_float), x.shape[0], C.c_float(eps), _p(y, C.c_float))
    return y


def rmsnorm_quant(x, gamma, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    g = np.ascontiguousarray(gamma, dtype=np.float32)
    q = np.empty(x.shape[0], dtype=np.int8)
    normed = np.empty_like(x)
    s = C.c_float()
    lib().orc_rmsnorm_quant(_p(x, C.c_float), _p(g, C.c_float), x.shape[0], C.c_float(eps),
                            _p(q, C.c_int8), C.byref(s), _p(normed, C.c_float))
    return q, np.float32(s.value), normed


def silu_mul_quant(g, u):
    g = np.ascontiguousarray(g, dtype=np.float32)
    u = np.ascontiguousarray(u, dtype=np.float32)
    q = np.empty(g.shape[0], dtype=np.int8)
    s = C.c_float()
    lib().orc_silu_mul_quant(_p(g, C.c_float), _p(u, C.c_float), g.shape[0], _p(q, C.c_int8), C.byref(s))
    return q, np.float32(s.value)


def relu2_mul_rmsnorm_quant(g, u, gamma, eps):
    g = np.ascontiguousarray(g, dtype=np.float32)
    u = np.ascontiguousarray(u, dtype=np.float32)
    gm = np.ascontiguousarray(gamma, dtype=np.float32)
    q = np.empty(g.shape[0], dtype=np.int8)
    s = C.c_float()
    lib().orc_relu2_mul_rmsnorm_quant(_p(g, C.c_float), _p(u, C.c_float), _p(gm, C.c_float),
                                      g.shape[0], C.c_float(eps), _p(q, C.c_int8), C.byref(s))
    return q, np.float32(s.value)


def rope_table(n_pos, head_dim, theta):
    t = np.empty((n_pos, head_dim // 2, 2), dtype=np.float32)
    lib().orc_rope_table(n_pos, head_dim, C.c_double(theta), _p(t, C.c_float))
    return t


def rope(v, n_heads, head_dim, table_row, neox):
    v = np.array(v, dtype=np.float32, copy=True)
    row = np.ascontiguousarray(table_row, dtype=np.float32)
    lib().orc_rope(_p(v, C.c_float), n_heads, head_dim, _p(row, C.c_float), int(neox))
    return v


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def attention(q, kc, vc, n_heads, n_kv, head_dim, smax, seq_len, twopass=False):
    q = np.ascontiguousarray(q, dtype=np.float32)
    kc = np.ascontiguousarray(kc, dtype=np.uint16)
    vc = np.ascontiguousarray(vc, dtype=np.uint16)
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    fn = lib().orc_attention_twopass if twopass else lib().orc_attention
    fn(_p(q, C.c_float), _p(kc, C.c_uint16), _p(vc, C.c_uint16), n_heads, n_kv, head_dim, smax,
       seq_len, _p(out, C.c_float))
    return out


def i2s_decode(raw, n_elems: int):
    """Restatement of the microsoft/BitNet i2_s decode (vendor/ntransformer/core/dequant.cpp:114-145,
    tools/convert_bitnet_to_packed.py:95-143): blocks of 128 elements in 32 bytes, byte p holds block positions
    p, p+32, p+64, p+96 with position p in the HIGH two bits; codes 0 -> -1, 1 -> 0, 2 -> +1, 3 -> 0; the fp32
    after the codes is the scale.  Returns (trits int8 [n_elems], scale)."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    blocks = raw[:n_elems // 4].reshape(-1, 32)
    lut = np.array([-1, 0, 1, 0], dtype=np.int8)
    out = np.empty((blocks.shape[0], 4, 32), dtype=np.int8)
    for g in range(4):
        out[:, g, :] = lut[(blocks >> (6 - 2 * g)) & 3]
    scale = float(raw[n_elems // 4:n_elems // 4 + 4].view(np.float32)[0])
    return out.reshape(-1), scale


def lm_head_bf16(embd, x):
    embd = np.ascontiguousarray(embd, dtype=np.uint16)
    x = np.ascontiguousarray(x, dtype=np.float32)
    V, H = embd.shape
    out = np.empty(V, dtype=np.float32)
    lib().orc_lm_head_bf16(_p(embd, C.c_uint16), _p(x, C.c_float), V, H, _p(out, C.c_float))
    return out


def argmax(v):
    v = np.ascontiguousarray(v, dtype=np.float32)
    return int(lib().orc_argmax(_p(v, C.c_float), v.shape[0]))


def expf(x: float) -> float:
    return float(lib().orc_expf(C.c_float(x)))


# ------------------------------------------------------------------ model
class Model:
    """Decode-forward oracle over weights given as v11-packed bytes."""

    def __init__(self, cfg: dict, threads: int = 0):
        self.cfg = dict(cfg)
        c = Cfg(arch=cfg["arch"], H=cfg["H"], F=cfg["F"], L=cfg["L"], V=cfg["V"], Nh=cfg["Nh"],
                Nkv=cfg["Nkv"], Hd=cfg["Hd"], Smax=cfg["Smax"], eps=cfg["eps"],
                rope_theta=cfg["rope_theta"], lm_head_packed=int(cfg.get("lm_head_packed", 0)),
                kv_f32=int(cfg.get("kv_f32", 0)), np_quant=int(cfg.get("np_quant", 0)))
        self._h = lib().orc_model_create(C.byref(c))
        lib().orc_model_set_threads(self._h, threads or (os.cpu_count() or 1))
        self._states = []

    def set_matrix(self, layer, which, packed_v11, scale):
        p = np.ascontiguousarray(packed_v11, dtype=np.uint8)
        rc = lib().orc_model_set_matrix(self._h, layer, which, p.ctypes.data, C.c_float(scale))
        assert rc == 0, rc

    def set_vector(self, layer, which, v):
        v = np.ascontiguousarray(v, dtype=np.float32)
        rc = lib().orc_model_set_vector(self._h, layer, which, v.ctypes.data)
        assert rc == 0, rc

    def set_embd(self, table_bf16):
        t = np.ascontiguousarray(table_bf16, dtype=np.uint16)
        rc = lib().orc_model_set_embd(self._h, t.ctypes.data)
        assert rc == 0, rc

    def new_state(self, batch=1):
        s = lib().orc_state_create(self._h, batch)
        self._states.append(s)
        return s

    def forward(self, state, seq, token, pos, want_logits=True, want_hidden=False):
        V, H = self.cfg["V"], self.cfg["H"]
        logits = np.empty(V, dtype=np.float32) if want_logits else None
        hidden = np.empty(H, dtype=np.float32) if want_hidden else None
        tok = lib().orc_forward_token(self._h, state, seq, int(token), int(pos),
                                      logits.ctypes.data if want_logits else None,
                                      hidden.ctypes.data if want_hidden else None)
        return tok, logits, hidden

    def layer_hidden(self, state, layer):
        out = np.empty(self.cfg["H"], dtype=np.float32)
        lib().orc_state_layer_hidden(state, layer, out.ctypes.data)
        return out

    def close(self):
        for s in self._states:
            lib().orc_state_destroy(s)
        self._states = []
        if self._h:
            lib().orc_model_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# -------------------------------------------------------------- reference
class Ref:
    """The unmodified reference CPU code (oracle/_ref/libter_ref.so)."""

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        L = C.CDLL(REF_SO)
        L.ref_ctx_create.restype = C.c_void_p
        L.ref_ctx_destroy.argtypes = [C.c_void_p]
        L.ref_tvmac.restype = C.c_uint64
        L.ref_tvmac.argtypes = [C.c_void_p]
        L.ref_reset_counters.argtypes = [C.c_void_p]
        L.ref_tensor_create.restype = C.c_void_p
        L.ref_tensor_create.argtypes = [C.c_void_p, C.c_size_t, C.c_float, C.c_int, C.c_int]
        L.ref_tensor_set_scale.argtypes = [C.c_void_p, C.c_float]
        L.ref_tensor_set_payload.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.ref_tensor_destroy.argtypes = [C.c_void_p]
        L.ref_mm_row.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.ref_mm_row_repeat.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int]
        L.ref_quantize.restype = C.c_float
        L.ref_quantize.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        if hasattr(L, "ref_tx_create"):
            L.ref_tx_create.restype = C.c_void_p
            L.ref_tx_create.argtypes = [C.c_int] * 9 + [C.c_float, C.c_double, C.c_uint64]
            L.ref_tx_destroy.argtypes = [C.c_void_p]
            L.ref_tx_forward_tokens.restype = C.c_double
            L.ref_tx_forward_tokens.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        self.L = L
        self.ctx = L.ref_ctx_create()

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def dequant_i2s(self, raw: np.ndarray, n_elems: int) -> np.ndarray:
        """nt::dequant_i2_s of the reference (vendor/ntransformer/core/dequant.cpp:114-145): raw = code bytes +
        32-byte trailer; returns n_elems floats (scale * {-1, 0, +1})."""
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        out = np.empty(n_elems, dtype=np.float32)
        self.L.ref_dequant_i2s.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        self.L.ref_dequant_i2s(raw.ctypes.data, n_elems, out.ctypes.data)
        return out

    def forward_token_seconds(self, cfg: dict, n_tokens: int = 3, first_pos: int = 27, seed: int = 1):
        """Times the reference's CPU decode forward (ter::tx::forward_token, src/tx/transformer.cpp:116-223)
        on a synthetic model of architecture `cfg` filled in place by the driver: returns (seconds per token,
        greedy tokens).  Single-threaded, as the reference is."""
        if not hasattr(self.L, "ref_tx_create"):
            raise RuntimeError("libter_ref.so was built without the forward driver")
        tx = self.L.ref_tx_create(int(cfg["arch"]), cfg["H"], cfg["F"], cfg["L"], cfg["V"], cfg["Nh"], cfg["Nkv"],
                                  cfg["Hd"], max(cfg.get("Smax", 64), first_pos + n_tokens), C.c_float(cfg["eps"]),
                                  C.c_double(cfg["rope_theta"]), seed)
        if not tx:
            raise MemoryError("reference model allocation failed")
        try:
            toks = np.zeros(n_tokens, np.int32)
            secs = float(self.L.ref_tx_forward_tokens(tx, 1, first_pos, n_tokens, toks.ctypes.data))
            if secs < 0:
                raise RuntimeError(f"reference forward_token failed ({secs})")
            return secs / n_tokens, toks
        finally:
            self.L.ref_tx_destroy(tx)

    def tensor(self, payload: np.ndarray, scale: float, rows: int, cols: int):
        p = np.ascontiguousarray(payload, dtype=np.int32)
        return self.L.ref_tensor_create(p.ctypes.data, p.size, C.c_float(scale), rows, cols)

    def free(self, t):
        self.L.ref_tensor_destroy(t)

    def mm_row_t(self, Xt, row, Wt, K, N):
        out = np.empty(N, dtype=np.float32)
        rc = self.L.ref_mm_row(self.ctx, Xt, row, Wt, K, N, out.ctypes.data)
        assert rc == 0
        return out

    def mm_row(self, X, x_scale, W, w_scale, row=0):
        """X int32 [rows][K] (or [K]), W int32 [K][N]."""
        W = np.ascontiguousarray(W, dtype=np.int32)
        K, N = W.shape
        X = np.ascontiguousarray(X, dtype=np.int32).reshape(-1, K)
        Xt = self.tensor(X, x_scale, X.shape[0], K)
        Wt = self.tensor(W, w_scale, K, N)
        try:
            return self.mm_row_t(Xt, row, Wt, K, N)
        finally:
            self.free(Xt)
            self.free(Wt)

    def mm_row_repeat(self, Xt, Wt, K, N, iters):
        out = np.empty(N, dtype=np.float32)
        rc = self.L.ref_mm_row_repeat(self.ctx, Xt, Wt, K, N, out.ctypes.data, iters)
        assert rc == 0
        return out

    def tvmac(self) -> int:
        return int(self.L.ref_tvmac(self.ctx))

    def reset_counters(self):
        self.L.ref_reset_counters(self.ctx)

    def quantize(self, x: np.ndarray, n_trits: int = 9):
        x = np.ascontiguousarray(x, dtype=np.float32)
        q = np.zeros(x.shape[0], dtype=np.int32)
        s = self.L.ref_quantize(x.ctypes.data, x.shape[0], n_trits, q.ctypes.data)
        return q, float(s)

    def __del__(self):
        try:
            self.L.ref_ctx_destroy(self.ctx)
        except Exception:
            pass
