"""ctypes binding over ``libter_b200.so`` (the C ABI of ``include/ter_b200.h``).

Host-side mirror of the reference's operator interface for the ternary matmul path:
``TerB200.install`` / ``gemv`` / ``gemv_acc`` / ``gemm`` take the same arguments, in the same
meaning, as ``mm_packed_dispatch(X, scale_x_dev, W{data, scale}, out, K, N, stream)``
(cuda/ter_cuda_forward_packed.cu:493-500) and ``mm_row`` (src/tx/forward.cpp:299-303).
Tensors are torch CUDA tensors used purely as device-memory holders; all arithmetic runs
in the library's own kernels.  Missing library => RuntimeError (never a CPU fallback).
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libter_b200.so")

FMT_V11, FMT_ROWMAJOR, FMT_I32 = 0, 1, 2
ACT_SILU, ACT_RELU2 = 1, 2
E_NULL, E_UNKNOWN, E_ALLOC, E_NARGS, E_SHAPE, E_FULL, E_NAME, E_CUDA, E_NCCL, E_STATE, E_TIMEOUT, E_VALUE, E_IO = \
    -1, -2, -3, -4, -5, -6, -7, -8, -9, -10, -11, -12, -13


class TerB200Error(RuntimeError):
    def __init__(self, code: int, what: str = ""):
        self.code = code
        msg = lib().ter_b200_strerror(code).decode() if _lib is not None else str(code)
        super().__init__(f"ter_b200 error {code} ({msg}) {what}".strip())


class OpCounts(C.Structure):
    _fields_ = [("total_ops", C.c_uint64), ("tvmac", C.c_uint64), ("tvadd", C.c_uint64),
                ("tvsub", C.c_uint64), ("tvmul", C.c_uint64)]


class ModelCfg(C.Structure):
    _fields_ = [("arch", C.c_int32), ("H", C.c_int32), ("F", C.c_int32), ("L", C.c_int32), ("V", C.c_int32),
                ("Nh", C.c_int32), ("Nkv", C.c_int32), ("Hd", C.c_int32), ("Smax", C.c_int32), ("eps", C.c_float),
                ("rope_theta", C.c_double), ("lm_head_packed", C.c_int32), ("max_batch", C.c_int32)]


def model_file_info(path: str) -> dict:
    """Header of an 'LLRT' / 'TERT' packed-model file (no GPU needed)."""
    c = ModelCfg()
    _check(load().ter_b200_model_file_info(os.fsencode(path), C.byref(c)), f"model_file_info {path}")
    return {k: getattr(c, k) for k, _ in ModelCfg._fields_}


class BlobHdr(C.Structure):
    _fields_ = [("magic", C.c_uint32), ("format", C.c_uint32), ("K", C.c_uint32), ("N", C.c_uint32),
                ("scale", C.c_float), ("reserved", C.c_uint32 * 3)]


BLOB_MAGIC = 0x54423257

_lib = None

# name -> (restype, argtypes); also the list the symbol-export test walks.
_VP, _CP, _I, _F, _SZ, _U64 = C.c_void_p, C.c_char_p, C.c_int, C.c_float, C.c_size_t, C.c_uint64
SIGNATURES = {
    "ter_b200_strerror": (C.c_char_p, [_I]),
    "ter_b200_create": (_VP, [_I]),
    "ter_b200_destroy": (None, [_VP]),
    "ter_b200_install_kernel": (_I, [_VP, _CP, _VP, _SZ]),
    "ter_b200_install_weight": (_I, [_VP, _CP, _VP, _I, _I, _I, _F]),
    "ter_b200_install_weight_dev": (_I, [_VP, _CP, _VP, _I, _I, _I, _F, _VP]),
    "ter_b200_remove_weight": (_I, [_VP, _CP]),
    "ter_b200_weight_info": (_I, [_VP, _CP, C.POINTER(_I), C.POINTER(_I), C.POINTER(_F)]),
    "ter_b200_call": (_I, [_VP, _CP, C.POINTER(C.c_int64), _SZ]),
    "ter_b200_op_counts": (None, [_VP, C.POINTER(OpCounts)]),
    "ter_b200_reset_counters": (None, [_VP]),
    "ter_b200_gemv": (_I, [_VP, _CP, _VP, _VP, _VP, _VP]),
    "ter_b200_gemv_acc": (_I, [_VP, _CP, _VP, _VP, _VP]),
    "ter_b200_gemv_group": (_I, [_VP, C.POINTER(_CP), _I, _VP, _VP, C.POINTER(_VP), _VP]),
    "ter_b200_gemv_multi": (_I, [_VP, _I, C.POINTER(_CP), C.POINTER(_VP), C.POINTER(_VP), C.POINTER(_VP), _VP]),
    "ter_b200_gemv_plan_create": (_I, [_VP, _I, C.POINTER(_CP), C.POINTER(_VP), C.POINTER(_VP), C.POINTER(_VP),
                                       C.POINTER(_I)]),
    "ter_b200_gemv_plan_launch": (_I, [_VP, _I, _VP]),
    "ter_b200_gemv_plan_destroy": (_I, [_VP, _I]),
    "ter_b200_norm_gemv_group": (_I, [_VP, C.POINTER(_CP), _I, _I, _VP, _VP, _VP, _F, C.POINTER(_VP), _I, _VP]),
    "ter_b200_gemv_host": (_I, [_VP, _CP, _VP, _F, _VP, _VP]),
    "ter_b200_gemv_host_batch": (_I, [_VP, _I, C.POINTER(_CP), C.POINTER(_VP), C.POINTER(_F), C.POINTER(_VP), _VP]),
    "ter_b200_sync": (_I, [_VP, _VP]),
    "ter_b200_gemm": (_I, [_VP, _CP, _VP, _VP, _I, _VP, _VP]),
    "ter_b200_gemm_acc": (_I, [_VP, _CP, _VP, _I, _VP, _VP]),
    "ter_b200_rmsnorm_quant": (_I, [_VP, _VP, _VP, _I, _I, _F, _VP, _VP, _VP, _VP]),
    "ter_b200_act_quant": (_I, [_VP, _I, _VP, _VP, _VP, _I, _I, _F, _VP, _VP, _VP]),
    "ter_b200_rope_kv": (_I, [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, C.c_double, _I, _VP, _VP, _VP]),
    "ter_b200_attention_scratch_floats": (_SZ, [_I, _I, _I, _I]),
    "ter_b200_attention": (_I, [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _VP, _SZ, _VP, _VP]),
    "ter_b200_attention_noalloc_max_floats": (_SZ, []),
    "ter_b200_attention_noalloc": (_I, [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _VP, _VP]),
    "ter_b200_lm_head_bf16": (_I, [_VP, _VP, _VP, _VP, _I, _I, _I, _VP]),
    "ter_b200_lm_head_bf16_tc": (_I, [_VP, _VP, _VP, _VP, _I, _I, _I, _VP, _SZ, _VP]),
    "ter_b200_lm_head_tc_scratch_bytes": (_SZ, [_I, _I]),
    "ter_b200_argmax": (_I, [_VP, _VP, _I, _I, _VP, _VP, _VP]),
    "ter_b200_model_create": (_I, [_VP, C.POINTER(ModelCfg)]),
    "ter_b200_model_set_matrix": (_I, [_VP, _I, _I, _VP, _I, _F]),
    "ter_b200_model_set_matrix_dev": (_I, [_VP, _I, _I, _VP, _I, _F]),
    "ter_b200_model_set_vector": (_I, [_VP, _I, _I, _VP]),
    "ter_b200_model_set_embd": (_I, [_VP, _VP]),
    "ter_b200_model_set_embd_dev": (_I, [_VP, _VP]),
    "ter_b200_model_load_file": (_I, [_VP, _CP, _I, _I, C.POINTER(ModelCfg)]),
    "ter_b200_model_file_info": (_I, [_CP, C.POINTER(ModelCfg)]),
    "ter_b200_convert_i2s": (_I, [_VP, _SZ, _I, _I, _VP, _VP]),
    "ter_b200_dump_op_stats": (_I, [_VP, _CP, _I, _I, _I, _I, _I, _I, _I, _I, _VP, _SZ]),
    "ter_b200_pick_kernel": (_I, [_VP, _I, _I, _I]),
    "ter_b200_kernel_name": (_CP, [_I]),
    "ter_b200_model_reset": (_I, [_VP, _I]),
    "ter_b200_decode_step": (_I, [_VP, _VP, _VP, _VP, _VP]),
    "ter_b200_model_logits": (_I, [_VP, _VP]),
    "ter_b200_model_hidden": (_I, [_VP, _VP]),
    "ter_b200_generate": (_I, [_VP, _VP, _I, _I, _I, _VP, _VP]),
    "ter_b200_last_generate_ms": (_F, [_VP]),
    "ter_b200_last_prefill_ms": (_F, [_VP]),
    "ter_b200_last_prompt_ms": (_F, [_VP]),
    "ter_b200_comm_unique_id": (_I, [_VP]),
    "ter_b200_comm_init": (_I, [_VP, _VP, _I, _I]),
    "ter_b200_comm_destroy": (None, [_VP]),
    "ter_b200_comm_rank": (_I, [_VP]),
    "ter_b200_comm_size": (_I, [_VP]),
    "ter_b200_capture_begin": (_I, [_VP, _VP]),
    "ter_b200_capture_end": (_I, [_VP, _VP, C.POINTER(_I)]),
    "ter_b200_graph_launch": (_I, [_VP, _I, _VP]),
    "ter_b200_graph_destroy": (_I, [_VP, _I]),
    "ter_b200_device_status": (_I, [_VP]),
    "ter_b200_selftest_exchange_timeout": (_I, [_VP]),
    "ter_b200_last_cuda_error": (_I, [_VP]),
    "ter_b200_set_option": (_I, [_VP, _CP, _I]),
    "ter_b200_launch_count": (_U64, [_VP]),
}


def load(path: str = LIB_PATH):
    """Load the shared library (building it in-tree first if it is absent and nvcc exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(path):
        try:
            from . import build as _b
            _b.build()
        except Exception as e:  # noqa: BLE001
            raise RuntimeError(
                f"ter_b200: CUDA library {path} is missing and could not be built ({e}); "
                "there is no CPU fallback") from e
    L = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)   # AttributeError here = ABI drift; let it surface
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def lib():
    return load()


def _check(rc: int, what: str = ""):
    if rc != 0:
        raise TerB200Error(rc, what)


_CUDA_STREAM_LEGACY = 0x1   # cudaStreamLegacy: the NULL stream named explicitly


def _stream_ptr(stream=None):
    """cudaStream_t of a torch stream (default: torch's current stream).  torch reports its default
    stream as 0, which the C ABI reads as "the handle's own stream"; name the legacy stream
    explicitly so that the library's launches stay ordered with torch's work."""
    import torch
    if stream is None:
        stream = torch.cuda.current_stream()
    return C.c_void_p(stream.cuda_stream or _CUDA_STREAM_LEGACY)


def convert_i2s(raw, N: int, K: int):
    """microsoft/BitNet i2_s tensor bytes (codes + 32-byte trailer) -> (v11 bytes [N/4][K], scale).  Host only."""
    import numpy as np
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    out = np.empty((N // 4, K), dtype=np.uint8)
    scale = C.c_float(0.0)
    rc = load().ter_b200_convert_i2s(raw.ctypes.data, raw.size, N, K, out.ctypes.data, C.byref(scale))
    if rc != 0:
        raise TerB200Error(rc, "convert_i2s")
    return out, float(scale.value)


class TerB200:
    """One handle = one GPU.  Mirrors the ter_k4 lifecycle: create, install, call, counters, destroy."""

    def __init__(self, device: int = 0):
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("ter_b200 needs a CUDA device; there is no CPU fallback")
        self.L = lib()
        self.device = device
        torch.cuda.set_device(device)
        self.h = self.L.ter_b200_create(device)
        if not self.h:
            raise RuntimeError(f"ter_b200_create({device}) failed")
        self._shapes = {}

    def _ck(self, rc: int, what: str = ""):
        if rc != 0:
            cu = self.L.ter_b200_last_cuda_error(self.h) if rc in (E_CUDA, E_ALLOC) else 0
            raise TerB200Error(rc, what + (f" [cudaError {cu}]" if cu else ""))

    # ---- lifecycle
    def close(self):
        if getattr(self, "h", None):
            self.L.ter_b200_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # ---- weights
    def install(self, name: str, data, fmt: int, K: int, N: int, scale: float):
        """data: numpy array (host) or torch CUDA tensor (device) in a boundary format."""
        import numpy as np
        import torch
        if isinstance(data, torch.Tensor) and data.is_cuda:
            d = data.contiguous()
            rc = self.L.ter_b200_install_weight_dev(self.h, name.encode(), C.c_void_p(d.data_ptr()), fmt, K, N,
                                                    scale, _stream_ptr())
        else:
            a = np.ascontiguousarray(data)
            rc = self.L.ter_b200_install_weight(self.h, name.encode(), C.c_void_p(a.ctypes.data), fmt, K, N, scale)
        _check(rc, f"install {name}")
        self._shapes[name] = (K, N)

    def install_blob(self, name: str, data, fmt: int, K: int, N: int, scale: float):
        """Same operation through the ter_k4-style blob verb."""
        import numpy as np
        a = np.ascontiguousarray(data)
        hdr = BlobHdr(BLOB_MAGIC, fmt, K, N, scale)
        blob = bytes(hdr) + a.tobytes()
        blob += b"\0" * (-len(blob) % 4)
        rc = self.L.ter_b200_install_kernel(self.h, name.encode(), blob, len(blob) // 4)
        _check(rc, f"install_kernel {name}")
        self._shapes[name] = (K, N)

    def remove(self, name: str):
        self._ck(self.L.ter_b200_remove_weight(self.h, name.encode()))
        self._shapes.pop(name, None)

    def weight_info(self, name: str):
        K, N, s = C.c_int(), C.c_int(), C.c_float()
        self._ck(self.L.ter_b200_weight_info(self.h, name.encode(), C.byref(K), C.byref(N), C.byref(s)))
        return K.value, N.value, s.value

    # ---- GEMV / GEMM
    def gemv(self, name: str, x, x_scale, out=None, stream=None):
        """x int8[K] cuda, x_scale float32[1] cuda -> float32[N]."""
        import torch
        K, N = self._shapes[name]
        if out is None:
            out = torch.empty(N, dtype=torch.float32, device=x.device)
        self._ck(self.L.ter_b200_gemv(self.h, name.encode(), C.c_void_p(x.data_ptr()), C.c_void_p(x_scale.data_ptr()),
                                    C.c_void_p(out.data_ptr()), _stream_ptr(stream)), f"gemv {name}")
        return out

    def gemv_acc(self, name: str, x, out=None, stream=None):
        import torch
        K, N = self._shapes[name]
        if out is None:
            out = torch.empty(N, dtype=torch.int32, device=x.device)
        self._ck(self.L.ter_b200_gemv_acc(self.h, name.encode(), C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()),
                                        _stream_ptr(stream)), f"gemv_acc {name}")
        return out

    def gemv_group(self, names, x, x_scale, outs=None, stream=None):
        import torch
        if outs is None:
            outs = [torch.empty(self._shapes[n][1], dtype=torch.float32, device=x.device) for n in names]
        arr_n = (C.c_char_p * len(names))(*[n.encode() for n in names])
        arr_o = (C.c_void_p * len(names))(*[o.data_ptr() for o in outs])
        self._ck(self.L.ter_b200_gemv_group(self.h, arr_n, len(names), C.c_void_p(x.data_ptr()),
                                          C.c_void_p(x_scale.data_ptr()), arr_o, _stream_ptr(stream)), "gemv_group")
        return outs

    def gemv_multi(self, names, xs, x_scales, outs=None, stream=None):
        """Independent GEMVs (own x, own K) in one launch."""
        import torch
        n = len(names)
        if outs is None:
            outs = [torch.empty(self._shapes[nm][1], dtype=torch.float32, device=xs[0].device) for nm in names]
        self._ck(self.L.ter_b200_gemv_multi(self.h, n, (C.c_char_p * n)(*[s.encode() for s in names]),
                                            (C.c_void_p * n)(*[t.data_ptr() for t in xs]),
                                            (C.c_void_p * n)(*[t.data_ptr() for t in x_scales]),
                                            (C.c_void_p * n)(*[t.data_ptr() for t in outs]), _stream_ptr(stream)),
                 "gemv_multi")
        return outs

    def gemv_plan(self, names, xs, x_scales, outs):
        """Sweep plan: all GEMVs in one launch per gemv_plan_launch(); tensors must stay alive."""
        n = len(names)
        pid = C.c_int(-1)
        self._ck(self.L.ter_b200_gemv_plan_create(self.h, n, (C.c_char_p * n)(*[s.encode() for s in names]),
                                                  (C.c_void_p * n)(*[t.data_ptr() for t in xs]),
                                                  (C.c_void_p * n)(*[t.data_ptr() for t in x_scales]),
                                                  (C.c_void_p * n)(*[t.data_ptr() for t in outs]), C.byref(pid)),
                 "gemv_plan_create")
        return pid.value

    def gemv_plan_launch(self, plan_id, stream=None):
        self._ck(self.L.ter_b200_gemv_plan_launch(self.h, plan_id, _stream_ptr(stream)), "gemv_plan_launch")

    def gemv_plan_destroy(self, plan_id):
        self._ck(self.L.ter_b200_gemv_plan_destroy(self.h, plan_id), "gemv_plan_destroy")

    def norm_gemv_group(self, names, x, gamma, eps, act=0, up=None, outs=None, accumulate=False, stream=None):
        """Fused quantiser + GEMV: x fp32[K] (gate for act != 0), returns fp32 outputs."""
        import torch
        if outs is None:
            outs = [torch.empty(self._shapes[n][1], dtype=torch.float32, device=x.device) for n in names]
        arr_n = (C.c_char_p * len(names))(*[n.encode() for n in names])
        arr_o = (C.c_void_p * len(names))(*[o.data_ptr() for o in outs])
        ptr = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
        self._ck(self.L.ter_b200_norm_gemv_group(self.h, arr_n, len(names), act, ptr(x), ptr(up), ptr(gamma),
                                               float(eps), arr_o, int(accumulate), _stream_ptr(stream)),
               "norm_gemv_group")
        return outs

    def gemv_host(self, name: str, x_host, x_scale: float, out_host, stream=None):
        """x_host int8[K], out_host float32[N]: (pinned) host torch tensors or numpy arrays. Asynchronous."""
        xp = x_host.data_ptr() if hasattr(x_host, "data_ptr") else x_host.ctypes.data
        op = out_host.data_ptr() if hasattr(out_host, "data_ptr") else out_host.ctypes.data
        self._ck(self.L.ter_b200_gemv_host(self.h, name.encode(), C.c_void_p(xp), float(x_scale), C.c_void_p(op),
                                         _stream_ptr(stream)), f"gemv_host {name}")

    def gemv_host_batch_plan(self, names, x_hosts, x_scales, out_hosts):
        """Pre-builds the argument arrays of ter_b200_gemv_host_batch (host tensors must stay alive)."""
        n = len(names)
        ptr = lambda t: t.data_ptr() if hasattr(t, "data_ptr") else t.ctypes.data  # noqa: E731
        return (n, (C.c_char_p * n)(*[s.encode() for s in names]), (C.c_void_p * n)(*[ptr(t) for t in x_hosts]),
                (C.c_float * n)(*[float(v) for v in x_scales]), (C.c_void_p * n)(*[ptr(t) for t in out_hosts]))

    def gemv_host_batch(self, plan, stream=None):
        n, names, xs, scales, outs = plan
        self._ck(self.L.ter_b200_gemv_host_batch(self.h, n, names, xs, scales, outs, _stream_ptr(stream)),
                 "gemv_host_batch")

    def sync(self, stream=None):
        self._ck(self.L.ter_b200_sync(self.h, _stream_ptr(stream)))

    def gemm(self, name: str, X, x_scales, out=None, stream=None):
        import torch
        K, N = self._shapes[name]
        M = X.shape[0]
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=X.device)
        self._ck(self.L.ter_b200_gemm(self.h, name.encode(), C.c_void_p(X.data_ptr()), C.c_void_p(x_scales.data_ptr()),
                                    M, C.c_void_p(out.data_ptr()), _stream_ptr(stream)), f"gemm {name}")
        return out

    def gemm_acc(self, name: str, X, out=None, stream=None):
        import torch
        K, N = self._shapes[name]
        M = X.shape[0]
        if out is None:
            out = torch.empty((M, N), dtype=torch.int32, device=X.device)
        self._ck(self.L.ter_b200_gemm_acc(self.h, name.encode(), C.c_void_p(X.data_ptr()), M,
                                        C.c_void_p(out.data_ptr()), _stream_ptr(stream)), f"gemm_acc {name}")
        return out

    def call(self, op: str, args):
        arr = (C.c_int64 * len(args))(*[int(a) for a in args])
        return self.L.ter_b200_call(self.h, op.encode(), arr, len(args))

    # ---- decode glue operators (fp32 torch CUDA tensors; rows = leading dimension)
    def rmsnorm_quant(self, x, gamma, eps, quant=True, want_normed=False, stream=None):
        import torch
        x2 = x.reshape(-1, x.shape[-1])
        rows, n = x2.shape
        q = torch.empty((rows, n), dtype=torch.int8, device=x.device) if quant else None
        sc = torch.empty(rows, dtype=torch.float32, device=x.device) if quant else None
        normed = torch.empty((rows, n), dtype=torch.float32, device=x.device) if (want_normed or not quant) else None
        ptr = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
        self._ck(self.L.ter_b200_rmsnorm_quant(self.h, ptr(x2), ptr(gamma), n, rows, float(eps), ptr(q), ptr(sc),
                                             ptr(normed), _stream_ptr(stream)), "rmsnorm_quant")
        return q, sc, normed

    def act_quant(self, act, gate, up, gamma, eps, stream=None):
        import torch
        g2 = gate.reshape(-1, gate.shape[-1])
        rows, n = g2.shape
        q = torch.empty((rows, n), dtype=torch.int8, device=gate.device)
        sc = torch.empty(rows, dtype=torch.float32, device=gate.device)
        self._ck(self.L.ter_b200_act_quant(self.h, act, C.c_void_p(g2.data_ptr()), C.c_void_p(up.data_ptr()),
                                         C.c_void_p(gamma.data_ptr()) if gamma is not None else None, n, rows,
                                         float(eps), C.c_void_p(q.data_ptr()), C.c_void_p(sc.data_ptr()),
                                         _stream_ptr(stream)), "act_quant")
        return q, sc

    def rope_kv(self, q, k, v, pos, Nh, Nkv, Hd, Smax, theta, neox, kcache, vcache, stream=None):
        B = pos.shape[0]
        self._ck(self.L.ter_b200_rope_kv(self.h, C.c_void_p(q.data_ptr()), C.c_void_p(k.data_ptr()),
                                       C.c_void_p(v.data_ptr()), C.c_void_p(pos.data_ptr()), B, Nh, Nkv, Hd, Smax,
                                       float(theta), int(neox), C.c_void_p(kcache.data_ptr()),
                                       C.c_void_p(vcache.data_ptr()), _stream_ptr(stream)), "rope_kv")

    def attention(self, q, kcache, vcache, pos, Nh, Nkv, Hd, Smax, scratch=None, out=None, stream=None):
        import torch
        B = pos.shape[0]
        need = self.L.ter_b200_attention_scratch_floats(B, Nh, Hd, Smax)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        if out is None:
            out = torch.empty((B, Nh * Hd), dtype=torch.float32, device=q.device)
        self._ck(self.L.ter_b200_attention(self.h, C.c_void_p(q.data_ptr()), C.c_void_p(kcache.data_ptr()),
                                         C.c_void_p(vcache.data_ptr()), C.c_void_p(pos.data_ptr()), B, Nh, Nkv, Hd,
                                         Smax, C.c_void_p(scratch.data_ptr()), scratch.numel(),
                                         C.c_void_p(out.data_ptr()), _stream_ptr(stream)), "attention")
        return out

    def attention_noalloc(self, q, kcache, vcache, pos, Nh, Nkv, Hd, Smax, out=None, stream=None):
        """Attention through the entry point that brings its own fixed scratch (no allocation inside
        the library; `out` is the caller's)."""
        import torch
        B = pos.shape[0]
        if out is None:
            out = torch.empty((B, Nh * Hd), dtype=torch.float32, device=q.device)
        self._ck(self.L.ter_b200_attention_noalloc(self.h, C.c_void_p(q.data_ptr()), C.c_void_p(kcache.data_ptr()),
                                                 C.c_void_p(vcache.data_ptr()), C.c_void_p(pos.data_ptr()), B, Nh,
                                                 Nkv, Hd, Smax, C.c_void_p(out.data_ptr()), _stream_ptr(stream)),
               "attention_noalloc")
        return out

    def lm_head_bf16(self, table, x, stream=None):
        import torch
        x2 = x.reshape(-1, x.shape[-1])
        B, H = x2.shape
        V = table.shape[0]
        logits = torch.empty((B, V), dtype=torch.float32, device=x.device)
        self._ck(self.L.ter_b200_lm_head_bf16(self.h, C.c_void_p(table.data_ptr()), C.c_void_p(x2.data_ptr()),
                                            C.c_void_p(logits.data_ptr()), V, H, B, _stream_ptr(stream)), "lm_head")
        return logits

    def lm_head_bf16_tc(self, table, x, stream=None):
        """The bf16 lm_head of a token batch on the tensor cores (rounding-level differences from lm_head_bf16)."""
        import torch
        x2 = x.reshape(-1, x.shape[-1])
        B, H = x2.shape
        V = table.shape[0]
        logits = torch.empty((B, V), dtype=torch.float32, device=x.device)
        nbytes = int(self.L.ter_b200_lm_head_tc_scratch_bytes(B, H))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        self._ck(self.L.ter_b200_lm_head_bf16_tc(self.h, C.c_void_p(table.data_ptr()), C.c_void_p(x2.data_ptr()),
                                               C.c_void_p(logits.data_ptr()), V, H, B, C.c_void_p(scratch.data_ptr()),
                                               nbytes, _stream_ptr(stream)), "lm_head_tc")
        return logits

    def argmax(self, logits, stream=None):
        import torch
        l2 = logits.reshape(-1, logits.shape[-1])
        B, V = l2.shape
        scratch = torch.empty(B * 256, dtype=torch.float32, device=logits.device)
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
        self._ck(self.L.ter_b200_argmax(self.h, C.c_void_p(l2.data_ptr()), V, B, C.c_void_p(scratch.data_ptr()),
                                      C.c_void_p(out.data_ptr()), _stream_ptr(stream)), "argmax")
        return out

    # ---- tensor parallelism
    def comm_init_from_torch(self):
        """Builds the library's NCCL communicator over the ranks of the default torch.distributed group
        (the id travels through torch's own broadcast; no data path goes through torch)."""
        import torch
        import torch.distributed as dist
        rank, world = dist.get_rank(), dist.get_world_size()
        buf = (C.c_uint8 * 128)()
        if rank == 0:
            _check(self.L.ter_b200_comm_unique_id(buf), "comm_unique_id")
        t = torch.tensor(list(bytes(buf)), dtype=torch.uint8, device=f"cuda:{self.device}" if dist.get_backend() == "nccl" else "cpu")
        dist.broadcast(t, 0)
        raw = bytes(t.cpu().tolist())
        self._ck(self.L.ter_b200_comm_init(self.h, raw, rank, world), "comm_init")

    # ---- decode forward
    def model_create(self, cfg: dict, max_batch: int = 1):
        c = ModelCfg(arch=cfg["arch"], H=cfg["H"], F=cfg["F"], L=cfg["L"], V=cfg["V"], Nh=cfg["Nh"], Nkv=cfg["Nkv"],
                     Hd=cfg["Hd"], Smax=cfg["Smax"], eps=cfg["eps"], rope_theta=cfg["rope_theta"],
                     lm_head_packed=int(cfg.get("lm_head_packed", 0)), max_batch=max_batch)
        self._ck(self.L.ter_b200_model_create(self.h, C.byref(c)), "model_create")
        self.model_cfg = dict(cfg, max_batch=max_batch)
        self._batch = 1

    def model_load_file(self, path: str, smax: int = 0, max_batch: int = 1) -> dict:
        """Creates and fills the model from an 'LLRT' / 'TERT' packed-model file; returns its configuration."""
        c = ModelCfg()
        self._ck(self.L.ter_b200_model_load_file(self.h, os.fsencode(path), smax, max_batch, C.byref(c)),
                 f"model_load_file {path}")
        cfg = {k: getattr(c, k) for k, _ in ModelCfg._fields_}
        self.model_cfg = dict(cfg)
        self._batch = 1
        return cfg

    def model_set_matrix(self, layer, which, data, fmt, scale):
        import numpy as np
        import torch
        if isinstance(data, torch.Tensor) and data.is_cuda:
            d = data.contiguous()
            rc = self.L.ter_b200_model_set_matrix_dev(self.h, layer, which, C.c_void_p(d.data_ptr()), fmt, float(scale))
        else:
            a = np.ascontiguousarray(data)
            rc = self.L.ter_b200_model_set_matrix(self.h, layer, which, C.c_void_p(a.ctypes.data), fmt, float(scale))
        _check(rc, f"model_set_matrix {layer}/{which}")

    def model_set_vector(self, layer, which, v):
        import numpy as np
        a = np.ascontiguousarray(v, dtype=np.float32)
        self._ck(self.L.ter_b200_model_set_vector(self.h, layer, which, C.c_void_p(a.ctypes.data)), "model_set_vector")

    def model_set_embd(self, table_bf16):
        import numpy as np
        import torch
        if isinstance(table_bf16, torch.Tensor) and table_bf16.is_cuda:
            rc = self.L.ter_b200_model_set_embd_dev(self.h, C.c_void_p(table_bf16.contiguous().data_ptr()))
        else:
            a = np.ascontiguousarray(table_bf16, dtype=np.uint16)
            rc = self.L.ter_b200_model_set_embd(self.h, C.c_void_p(a.ctypes.data))
        _check(rc, "model_set_embd")

    def model_reset(self, batch=1):
        self._ck(self.L.ter_b200_model_reset(self.h, batch), "model_reset")
        self._batch = batch

    def decode_step(self, tokens=None, pos=None, want_next=True, stream=None):
        import numpy as np
        B = self._batch
        t = np.ascontiguousarray(tokens, dtype=np.int32) if tokens is not None else None
        p = np.ascontiguousarray(pos, dtype=np.int32) if pos is not None else None
        nxt = np.empty(B, dtype=np.int32) if want_next else None
        self._ck(self.L.ter_b200_decode_step(self.h, C.c_void_p(t.ctypes.data) if t is not None else None,
                                           C.c_void_p(p.ctypes.data) if p is not None else None,
                                           C.c_void_p(nxt.ctypes.data) if want_next else None,
                                           _stream_ptr(stream)), "decode_step")
        return nxt

    def model_logits(self):
        import numpy as np
        out = np.empty((self._batch, self.model_cfg["V"]), dtype=np.float32)
        self._ck(self.L.ter_b200_model_logits(self.h, C.c_void_p(out.ctypes.data)), "model_logits")
        return out

    def model_hidden(self):
        import numpy as np
        out = np.empty((self._batch, self.model_cfg["H"]), dtype=np.float32)
        self._ck(self.L.ter_b200_model_hidden(self.h, C.c_void_p(out.ctypes.data)), "model_hidden")
        return out

    def generate(self, prompts, n_gen, stream=None):
        """prompts int32 [batch][n_prompt] -> int32 [batch][n_gen] greedy tokens."""
        import numpy as np
        p = np.ascontiguousarray(prompts, dtype=np.int32)
        if p.ndim == 1:
            p = p[None, :]
        B, n_prompt = p.shape
        out = np.empty((B, n_gen), dtype=np.int32)
        self._ck(self.L.ter_b200_generate(self.h, C.c_void_p(p.ctypes.data), B, n_prompt, n_gen,
                                        C.c_void_p(out.ctypes.data), _stream_ptr(stream)), "generate")
        self._batch = B
        return out

    def last_generate_ms(self) -> float:
        return float(self.L.ter_b200_last_generate_ms(self.h))

    def last_prompt_ms(self) -> float:
        return float(self.L.ter_b200_last_prompt_ms(self.h))

    def last_prefill_ms(self) -> float:
        return float(self.L.ter_b200_last_prefill_ms(self.h))

    # ---- CUDA graphs
    def capture(self, fn, stream=None):
        """Record the launches fn() makes through this handle into a CUDA graph; returns its id."""
        import torch
        s = stream or torch.cuda.Stream()
        gid = C.c_int(-1)
        with torch.cuda.stream(s):
            self._ck(self.L.ter_b200_capture_begin(self.h, _stream_ptr(s)), "capture_begin")
            try:
                fn()
            finally:
                rc = self.L.ter_b200_capture_end(self.h, _stream_ptr(s), C.byref(gid))
            _check(rc, "capture_end")
        return gid.value

    def graph_launch(self, gid: int, stream=None):
        self._ck(self.L.ter_b200_graph_launch(self.h, gid, _stream_ptr(stream)), "graph_launch")

    def graph_destroy(self, gid: int):
        self._ck(self.L.ter_b200_graph_destroy(self.h, gid))

    # ---- counters / status
    def op_counts(self) -> dict:
        c = OpCounts()
        self.L.ter_b200_op_counts(self.h, C.byref(c))
        return {k: getattr(c, k) for k, _ in OpCounts._fields_}

    def reset_counters(self):
        self.L.ter_b200_reset_counters(self.h)

    def launch_count(self) -> int:
        return int(self.L.ter_b200_launch_count(self.h))

    def device_status(self) -> int:
        return self.L.ter_b200_device_status(self.h)

    def pick_kernel(self, M: int, K: int, N: int) -> str:
        """Name of the kernel the library's dispatch rule picks for M rows against a K x N weight."""
        k = self.L.ter_b200_pick_kernel(self.h, M, K, N)
        if k < 0:
            raise TerB200Error(k, "pick_kernel")
        return self.L.ter_b200_kernel_name(k).decode()

    def op_stats_report(self, label: str, cfg: dict, n_forwards: int) -> str:
        buf = C.create_string_buffer(4096)
        self.L.ter_b200_dump_op_stats(self.h, label.encode(), cfg["H"], cfg["F"], cfg["Nh"], cfg["Nkv"], cfg["Hd"],
                                      cfg["L"], cfg["V"], n_forwards, buf, len(buf))
        return buf.value.decode()

    def selftest_exchange_timeout(self):
        self._ck(self.L.ter_b200_selftest_exchange_timeout(self.h), "selftest_exchange_timeout")

    def set_option(self, key: str, value: int):
        self._ck(self.L.ter_b200_set_option(self.h, key.encode(), int(value)), f"set_option {key}")
