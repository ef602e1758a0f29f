"""Loading the kernel library and calling its entry points with torch tensors.

The library is plain C ABI (``extern "C"``): raw device pointers, sizes and a stream. It is loaded with ctypes from
the in-tree build folder; a missing or unbuildable library is an error, never a fallback to other code. Each
wrapper below checks what the kernel itself does not (contiguity, dtypes, size limits) and raises on a failed
launch.
"""
from __future__ import annotations

import ctypes
import functools
from ctypes import c_int, c_float, c_void_p, c_longlong
from typing import Optional

import torch

from . import build as _build

F32, BF16 = 0, 1
PAGE = 64                     # positions per cache page (KB_PAGE in csrc/common.cuh)

ST_BAD_TOKEN, ST_BAD_PAGE, ST_WAIT_TIMEOUT, ST_BAD_ROW = 1, 2, 4, 8

_lib = None


class KernelError(RuntimeError):
    pass


_SIGS = {
    "kb_embed": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "kb_logit_post": [c_void_p, c_longlong, c_float, c_float, c_void_p],
    "kb_add_rmsnorm": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p,
                       c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "kb_gemm_simt": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                     c_void_p],
    "kb_rope_store": [c_void_p, c_int, c_int, c_longlong, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p,
                      c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p,
                      c_void_p, c_void_p],
    "kb_rope_table": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "kb_attn_generic": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                        c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p,
                        c_void_p, c_int],
    "kb_gate_mul": [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_longlong, c_int, c_void_p, c_int, c_int, c_int,
                    c_void_p],
    "kb_gated_rmsnorm": [c_void_p, c_int, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_longlong, c_int, c_void_p,
                         c_int, c_int, c_int, c_int, c_void_p],
    "kb_latent_prep": [c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                       c_float, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                       c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "kb_latent_qrope": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
                        c_int, c_int, c_int, c_void_p],
    "kb_head_gemm": [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                     c_int, c_void_p, c_int, c_int, c_longlong, c_int, c_void_p, c_int],
    "kb_decay_chunked": [c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "kb_decay_scan": [c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                      c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "kb_add_layernorm": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int,
                         c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "kb_residual_add": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_longlong, c_void_p],
    "kb_norm_rope_store": [c_void_p, c_int, c_int, c_longlong, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                           c_float, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                           c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "kb_moe_topk": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int],
    "kb_sinusoid_add": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "kb_mix_cat": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "kb_short_conv": [c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                      c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                      c_void_p],
    "kb_delta_rule": [c_void_p, c_int, c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p,
                      c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                      c_int, c_void_p],
    "kb_delta_chunked": [c_void_p, c_int, c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p,
                         c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                         c_void_p, c_int, c_void_p, c_int, c_void_p],
    "kb_head_norm_gate": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_int, c_int, c_longlong,
                          c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p],
    "kb_min_gru": [c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                   c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p],
    "kb_branch_norm_mean": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int,
                            c_void_p],
    "kb_moe_gate_mul": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "kb_row_gate": [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
    "kb_sigattn_prep": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_float,
                        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                        c_void_p, c_void_p],
    "kb_sigmoid_attn": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                        c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "kb_sigattn_decode": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                          c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "kb_sigattn_tc": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                      c_float, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "kb_moe_plan": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "kb_moe_gemm_tile": [],
    "kb_moe_gemm_tc_tile": [],
    "kb_moe_gemm_tc": [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_longlong, c_int,
                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                       c_void_p, c_void_p, c_int, c_float, c_float],
    "kb_moe_gather": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
    "kb_moe_gemm": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_int,
                    c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "kb_swiglu": [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int],
    "kb_gemm_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                   c_longlong, c_void_p, c_void_p, c_int, c_int, c_float, c_float],
    "kb_gemm_tc_splits": [c_int, c_int],
    "kb_rope_table_min_rows": [],
    "kb_gemm_pair": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                     c_void_p, c_int, c_void_p, c_void_p, c_float, c_float],
    "kb_gemm_swiglu_decode": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_int, c_float, c_float],
    "kb_attn_mma": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                    c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                    c_int, c_void_p],
    "kb_attn_decode_rope": [c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_void_p,
                            c_int, c_int, c_int, c_void_p, c_void_p],
    "kb_attn_tc": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                   c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int],
    "kb_sample": [c_void_p, c_longlong, c_int, c_int, c_float, c_int, c_float, c_float, c_int, c_void_p, c_void_p,
                  c_void_p],
    "kb_penalize": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_float, c_void_p],
    "kb_wait_selftest": [ctypes.c_ulonglong, c_void_p, c_void_p, c_void_p],
    "kb_headnorm_rope_store": [c_void_p, c_int, c_int, c_longlong, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                               c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p,
                               c_void_p],
    "kb_diff_combine": [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                        c_float, c_void_p],
    "kb_head_gate_mul": [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_longlong, c_int, c_void_p, c_int, c_int,
                         c_int, c_int, c_void_p],
    "kb_postnorm_add": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p,
                        c_int, c_int, c_int, c_void_p],
    "kb_cast_rows": [c_void_p, c_void_p, c_int, c_longlong, c_void_p],
    "kb_glu_clamp": [c_void_p, c_int, c_int, c_longlong, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                     c_float, c_void_p],
    "kb_moe_route": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "kb_moe_identity": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                        c_void_p],
}


def load(verbose: bool = True):
    """build (when needed) and load the kernel library; raises when that is not possible"""
    global _lib
    if _lib is not None:
        return _lib if _timing is None else _timing
    path = _build.library_path(build=True, verbose=verbose)
    lib = ctypes.CDLL(path)
    for name, args in _SIGS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            raise KernelError("kindi_b200: the kernel library %s lacks %s" % (path, name))
        fn.argtypes = args
        fn.restype = c_int
    lib.kb_set_pdl.argtypes = [c_int]
    lib.kb_set_pdl.restype = None
    lib._path = path
    _lib = lib
    return lib


# ----------------------------------------------------------------------------------------------- per-kernel timing
_timing = None

# where an entry point's product sizes stand among its arguments (N, K), for the label of a timed launch
_GEMM_NK = {"kb_gemm_tc": (5, 6), "kb_gemm_pair": (5, 6), "kb_gemm_simt": (7, 8), "kb_gemm_swiglu_decode": (4, 5)}


class KernelTiming:
    """``with KernelTiming() as t: engine.step(...)``: every launch of the library inside the block is bracketed by
    CUDA events on the launching stream; ``t.summary()`` gives, per kind of launch (entry point, with the product's
    sizes for matrix products), the number of launches and the device time in microseconds. Meant for steps that are
    issued launch by launch (a recorded step is one launch to the host); the events themselves cost the device a
    microsecond or two per launch, so compare shares."""

    def __init__(self):
        self.records = []

    def __getattr__(self, name):                       # stands in for the library while timing is on
        fn = getattr(_lib, name)
        if not name.startswith("kb_") or name in ("kb_set_pdl", "kb_gemm_tc_splits", "kb_rope_table_min_rows",
                                                  "kb_moe_gemm_tile", "kb_moe_gemm_tc_tile"):
            return fn

        def timed(*args):
            label = name[3:]
            if name in _GEMM_NK:
                n, k = _GEMM_NK[name]
                label += " %dx%d" % ((2 * args[n], args[k]) if name == "kb_gemm_swiglu_decode" else (args[n], args[k]))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = fn(*args)
            e1.record()
            self.records.append((label, e0, e1))
            return rc
        return timed

    def __enter__(self):
        global _timing
        load()
        _timing = self
        return self

    def __exit__(self, *exc):
        global _timing
        _timing = None
        return False

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        for label, e0, e1 in self.records:
            d = out.setdefault(label, {"launches": 0, "us": 0.0})
            d["launches"] += 1
            d["us"] += e0.elapsed_time(e1) * 1000.0
        return {k: {"launches": v["launches"], "us": round(v["us"], 1)} for k, v in out.items()}


def set_pdl(on: bool) -> None:
    """launch kernels with programmatic dependent launch (the default) or strictly one after another"""
    load().kb_set_pdl(1 if on else 0)


def library_file() -> str:
    return load()._path


_launches = 0


def launch_count() -> int:
    """kernels of this library launched so far (replays of a recorded step count the launches they hold)"""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(rc: int, what: str) -> None:
    global _launches
    _launches += 1
    if rc != 0:
        raise KernelError("kindi_b200: launching %s failed with CUDA error %d (%s)"
                          % (what, rc, _err_name(rc)))


def _err_name(rc: int) -> str:
    try:
        return torch.cuda.cudart().cudaGetErrorString(rc)      # type: ignore[attr-defined]
    except Exception:                                          # noqa: BLE001
        return "?"


def dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError("kindi_b200: tensors must be float32 or bfloat16, found %s" % t.dtype)


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None) or torch.cuda.current_device


def _stream():
    """the current stream's handle (asked of torch directly: building a Stream object costs several microseconds,
    which a step of a hundred launches feels)"""
    if _raw_stream is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("kindi_b200: the kernels run on the GPU only; a tensor lives on %s" % t.device)


# ----------------------------------------------------------------------------------------------- wrappers
def embed(table: torch.Tensor, tok: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
          scale: float = 1.0) -> None:
    """out[t] (float32 [T, E]) = table[tok[t]] * scale"""
    _need_cuda(table, tok, out)
    T, E = out.shape
    assert table.is_contiguous() and out.is_contiguous() and out.dtype == torch.float32 and tok.dtype == torch.int32
    _check(load().kb_embed(_p(table), dt(table), _p(tok), _p(out), T, E, table.shape[0], float(scale), _p(status),
                           _stream()), "embed")


def wait_selftest(status: torch.Tensor, limit_ns: int = 1_000_000):
    """run the library's bounded wait on a barrier that nothing arrives at: it gives up after ``limit_ns`` (at most a
    tenth of a second), sets ST_WAIT_TIMEOUT in ``status`` and the kernel ends. Returns (timed out, nanoseconds waited)
    once the kernel has finished"""
    _need_cuda(status)
    out = torch.zeros(2, dtype=torch.int64, device=status.device)
    _check(load().kb_wait_selftest(int(limit_ns), _p(out), _p(status), _stream()), "wait_selftest")
    r = out.tolist()
    return bool(r[0]), int(r[1])


def logit_post(logits: torch.Tensor, scale: float = 1.0, softcap: float = 0.0) -> None:
    """logits (float32, contiguous) *= scale, then softcap * tanh(logits / softcap) when softcap > 0; in place"""
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    _check(load().kb_logit_post(_p(logits), logits.numel(), float(scale), float(softcap), _stream()), "logit_post")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor], write_back: bool, status: torch.Tensor,
                branch_scale: Optional[torch.Tensor] = None) -> None:
    """x (float32 [T, E]) + sum of delta ([S, T, E] float32) -> RMS norm * w -> out ([R, E]); rows int32 or None.
    ``branch_scale`` ([E], the gains' dtype): the summed delta is multiplied by it, column by column, before the add"""
    _need_cuda(x, delta, w, out, rows, branch_scale)
    if branch_scale is not None:
        assert branch_scale.dtype == w.dtype and branch_scale.is_contiguous() and branch_scale.numel() == x.shape[1]
    T, E = x.shape
    n_out = out.shape[0]
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and w.shape == (E,)
    nd, stride = 0, 0
    if delta is not None:
        assert delta.dtype == torch.float32 and delta.is_contiguous() and delta.shape[1:] == (T, E)
        nd, stride = delta.shape[0], T * E
    if rows is None:
        assert n_out == T
    else:
        assert rows.dtype == torch.int32 and rows.numel() == n_out
    if E * 4 > 200 * 1024:
        raise KernelError("kindi_b200: RMS norm supports a width up to 51200, found %d" % E)
    _check(load().kb_add_rmsnorm(_p(x), _p(delta), nd, stride, _p(w), dt(w), float(eps), _p(out), dt(out), _p(rows),
                                 n_out, T, E, 1 if write_back else 0, _p(status), _stream(),
                                 _p(branch_scale) if delta is not None else None), "add_rmsnorm")


def add_layernorm(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, b: torch.Tensor, eps: float,
                  out: torch.Tensor, rows: Optional[torch.Tensor], write_back: bool, status: torch.Tensor) -> None:
    """x (float32 [T, E]) + sum of delta ([S, T, E] float32) -> (v - mean) / sqrt(var + eps) * w + b -> out ([R, E]);
    rows int32 or None"""
    _need_cuda(x, delta, w, b, out, rows)
    T, E = x.shape
    n_out = out.shape[0]
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and w.shape == (E,) == b.shape
    assert w.dtype == b.dtype and w.is_contiguous() and b.is_contiguous()
    nd, stride = 0, 0
    if delta is not None:
        assert delta.dtype == torch.float32 and delta.is_contiguous() and delta.shape[1:] == (T, E)
        nd, stride = delta.shape[0], T * E
    if rows is None:
        assert n_out == T
    else:
        assert rows.dtype == torch.int32 and rows.numel() == n_out
    if E > 51200:
        raise KernelError("kindi_b200: layer norm supports a width up to 51200, found %d" % E)
    _check(load().kb_add_layernorm(_p(x), _p(delta), nd, stride, _p(w), _p(b), dt(w), float(eps), _p(out), dt(out),
                                   _p(rows), n_out, T, E, 1 if write_back else 0, _p(status), _stream()),
           "add_layernorm")


def residual_add(x: torch.Tensor, delta: Optional[torch.Tensor], extra: Optional[torch.Tensor]) -> None:
    """x (float32 [T, E]) += sum of delta ([S, T, E] float32, in order) + extra ([T, E] float32); in place"""
    _need_cuda(x, delta, extra)
    assert x.dtype == torch.float32 and x.is_contiguous()
    nd, stride = 0, 0
    if delta is not None:
        assert delta.dtype == torch.float32 and delta.is_contiguous() and delta.shape[1:] == x.shape
        nd, stride = delta.shape[0], x.numel()
    if extra is not None:
        assert extra.dtype == torch.float32 and extra.is_contiguous() and extra.shape == x.shape
    _check(load().kb_residual_add(_p(x), _p(delta), nd, stride, _p(extra), x.numel(), _stream()), "residual_add")


def norm_rope_store(qkv: torch.Tensor, qout: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor],
                    eps: float, nq_true: int, nk_true: int, inv_freq: torch.Tensor, rot: int, pos, seq, slot, nh: int,
                    nkv: int, nkv_store: int, hd: int, pool: Optional[torch.Tensor], table: torch.Tensor, n_pages: int,
                    status: torch.Tensor) -> None:
    """``rope_store`` with a norm in front: the query part and the key part of a row are each divided by their root
    mean square over all their heads (``sqrt(sum / n_true + eps)``) and multiplied by the gains ``wq`` ([nh hd]) and
    ``wk`` ([nkv hd]) before the rotation. qkv: rows or 32-bit planes of [q heads | k heads | v heads]"""
    _need_cuda(qkv, qout, wq, wk, inv_freq, pool, table)
    planes = qkv.shape[0] if qkv.dim() == 3 else 1
    T = qkv.shape[-2]
    assert qkv.stride(-1) == 1 and qkv.shape[-1] == (nh + 2 * nkv) * hd and qout.stride(1) == 1
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() >= max(1, rot // 2) and rot % 2 == 0 and rot <= hd
    wd = F32
    if wq is not None:
        assert wq.dtype == wk.dtype and wq.numel() == nh * hd and wk.numel() == nkv * hd
        assert wq.is_contiguous() and wk.is_contiguous()
        wd = dt(wq)
    if nkv_store:
        assert pool is not None and pool.dtype == qout.dtype and pool.is_contiguous() and nkv_store == nkv
    pstride = qkv.stride(0) if qkv.dim() == 3 else 0
    rc = load().kb_norm_rope_store(_p(qkv), dt(qkv), planes, pstride, qkv.stride(-2), _p(qout), dt(qout),
                                   qout.stride(0), _p(wq), _p(wk), wd, float(eps), int(nq_true), int(nk_true),
                                   _p(inv_freq), rot, _p(pos), _p(seq), _p(slot), T, nh, nkv, nkv_store, hd,
                                   _p(pool), _p(table), table.stride(0), n_pages, _p(status), _stream())
    _check(rc, "norm_rope_store")


ACT = {"none": 0, "relu2": 1, "silu": 2, "gelu_tanh": 3}
# what a gated feed-forward's gate may pass through inside a product's epilogue; "glu_clamp" (with ``act_params`` =
# (limit, alpha)): g' sigmoid(alpha g') (u' + 1), gate clamped from above, up from both sides
GATE_ACT = {"silu": ACT["silu"], "gelu_tanh": ACT["gelu_tanh"], "glu_clamp": 4}


def _gate_params(act: str, act_params):
    if act == "glu_clamp":
        return float(act_params[0]), float(act_params[1])
    return 0.0, 0.0


def _planes_of(g: torch.Tensor):
    """(number of planes, plane stride, row stride) of rows [T, N] or 32-bit planes [S, T, N]"""
    if g.dim() == 3:
        assert g.dtype == torch.float32 and g.stride(2) == 1
        return g.shape[0], g.stride(0), g.stride(1)
    assert g.stride(1) == 1
    return 1, 0, g.stride(0)


def gate_mul(a: torch.Tensor, g: torch.Tensor, out: torch.Tensor) -> None:
    """out[t][c] = a[t][c] * sigmoid(g[t][c]); ``g``: rows [T, N] or 32-bit planes [S, T, N] (views are fine)"""
    _need_cuda(a, g, out)
    T, N = a.shape
    n_planes, pstride, ldg = _planes_of(g)
    assert g.shape[-2:] == (T, N) and out.shape == (T, N) and a.stride(1) == 1 and out.stride(1) == 1
    assert out.dtype == a.dtype
    _check(load().kb_gate_mul(_p(a), dt(a), a.stride(0), _p(g), dt(g), n_planes, pstride, ldg, _p(out), out.stride(0),
                              T, N, _stream()), "gate_mul")


def gated_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, g: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w * sigmoid(g[t]); x float32 [T, N]; ``g`` rows or 32-bit planes"""
    _need_cuda(x, w, g, out)
    T, N = x.shape
    assert x.dtype == torch.float32 and x.stride(1) == 1 and w.numel() == N and w.is_contiguous()
    assert out.shape == (T, N) and out.stride(1) == 1
    n_planes, pstride, ldg = _planes_of(g) if g is not None else (1, 0, 0)
    if g is not None:
        assert g.shape[-2:] == (T, N)
    _check(load().kb_gated_rmsnorm(_p(x), x.stride(0), _p(w), dt(w), float(eps), _p(g), dt(g) if g is not None else F32,
                                   n_planes, pstride, ldg, _p(out), dt(out), out.stride(0), T, N, _stream()),
           "gated_rmsnorm")


def latent_prep(a: torch.Tensor, q_rank: int, kv_rank: int, rot: int, wq: torch.Tensor, wkv: torch.Tensor, eps: float,
                freq: torch.Tensor, mult: float, pos, seq, slot, cq: torch.Tensor, head_dim: int, pool: torch.Tensor,
                table: torch.Tensor, n_pages: int, status: torch.Tensor) -> None:
    """``a``: rows or 32-bit planes of [query latent | key/value latent | rotated key part | ...]. Writes the RMS-normed
    query latent to ``cq`` and stores, at each row's position of its sequence's pages, one key head [normed latent |
    rotated part | 0] and one value head [normed latent | 0] of ``head_dim`` elements. The rotation pairs element 2i
    with 2i + 1, by pos * freq[i], cosine and sine times ``mult``"""
    _need_cuda(a, wq, wkv, freq, cq, pool, table)
    n_planes, pstride, ld = _planes_of(a)
    T = a.shape[-2]
    assert a.shape[-1] >= q_rank + kv_rank + rot and wq.dtype == wkv.dtype and wq.numel() == q_rank
    assert wkv.numel() == kv_rank and wq.is_contiguous() and wkv.is_contiguous()
    assert freq.dtype == torch.float32 and freq.numel() >= max(1, rot // 2) and freq.is_contiguous()
    assert cq.shape == (T, q_rank) and cq.stride(1) == 1 and pool.dtype == cq.dtype and pool.is_contiguous()
    assert pool.shape[-1] == head_dim and pool.shape[-3] == 1
    _check(load().kb_latent_prep(_p(a), dt(a), n_planes, pstride, ld, q_rank, kv_rank, rot, _p(wq), _p(wkv), dt(wq),
                                 float(eps), _p(freq), float(mult), _p(pos), _p(seq), _p(slot), _p(cq), dt(cq),
                                 cq.stride(0), T, head_dim, _p(pool), _p(table), table.stride(0), n_pages, _p(status),
                                 _stream()), "latent_prep")


def latent_qrope(q: torch.Tensor, dim: int, rot: int, freq: torch.Tensor, mult: float, pos, out: torch.Tensor,
                 at: int, head_dim: int, n_heads: int) -> None:
    """q rows [T, n_heads (dim + rot)]: each head's last ``rot`` elements, rotated (pairs 2i, 2i + 1), go to
    out[t][h][at : at + rot]; out[t][h][at + rot : head_dim] = 0"""
    _need_cuda(q, freq, out)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype and q.shape[1] == n_heads * (dim + rot)
    assert out.shape == (T, n_heads * head_dim) and freq.dtype == torch.float32
    _check(load().kb_latent_qrope(_p(q), dt(q), q.stride(0), dim, rot, _p(freq), float(mult), _p(pos), _p(out),
                                  out.stride(0), at, head_dim, T, n_heads, _stream()), "latent_qrope")


def head_gemm(a: torch.Tensor, a_head_stride: int, w: torch.Tensor, out: torch.Tensor, out_head_stride: int,
              gate: Optional[torch.Tensor] = None, tensor_cores: bool = True) -> None:
    """per head h: out[t][h * out_head_stride + n] = sum_k a[t][h * a_head_stride + k] * w[h][n][k]; w [H, N, K].
    ``gate`` (rows or 32-bit planes [.., T, H * N]): the result is multiplied by its logistic function. bf16 operands
    whose rows are 16-byte aligned (K, strides multiples of 8) run on the tensor cores unless ``tensor_cores`` is
    False; everything else takes 32-bit multiply-adds in a fixed order"""
    _need_cuda(a, w, out, gate)
    H, N, Kd = w.shape
    M = a.shape[0]
    assert a.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous() and out.dtype == a.dtype
    assert a.shape[1] >= (H - 1) * a_head_stride + Kd and out.shape[1] >= (H - 1) * out_head_stride + N
    n_planes, pstride, ldg = _planes_of(gate) if gate is not None else (1, 0, 0)
    if gate is not None:
        assert gate.shape[-2:] == (M, H * N)
    _check(load().kb_head_gemm(_p(a), dt(a), a.stride(0), a_head_stride, _p(w), dt(w), _p(out), out.stride(0),
                               out_head_stride, M, N, Kd, H, _p(gate), dt(gate) if gate is not None else F32, n_planes,
                               pstride, ldg, _stream(), 1 if tensor_cores else 0), "head_gemm")


def decay_scan(a: torch.Tensor, B: int, H: int, d: int, dv: int, decay: torch.Tensor, q_start, slot,
               state: torch.Tensor, out: torch.Tensor, chunk: int = 0, max_rows: int = 0) -> None:
    """linear attention with a decay per head over the packed rows of ``B`` sequences: ``a`` rows or 32-bit planes of
    [q (H d) | k (H d) | v (H dv) | ...] (silu is applied here); ``state`` float32 [slots, H, dv, d] is read and
    written; ``out`` float32 [T, H dv]. ``chunk`` > 0: the form for long prompts that works on a sequence's runs of
    ``chunk`` tokens side by side (``max_rows``: the most rows a sequence brings, or an upper bound); its sums differ
    from the token-by-token form's by rounding"""
    _need_cuda(a, decay, state, out)
    n_planes, pstride, ld = _planes_of(a)
    assert a.shape[-1] >= 2 * H * d + H * dv and decay.dtype == torch.float32 and decay.numel() == H
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (H, dv, d)
    assert out.dtype == torch.float32 and out.stride(1) == 1 and out.shape[1] == H * dv
    if d > 256:
        raise KernelError("kindi_b200: linear attention supports key sizes up to 256, found %d" % d)
    if chunk > 0:
        nc = max(1, -(-int(max_rows) // chunk))
        scratch = torch.empty((B * H * (nc + 1), dv, d), dtype=torch.float32, device=out.device)
        _check(load().kb_decay_chunked(_p(a), dt(a), n_planes, pstride, ld, B, H, d, dv, _p(decay), _p(q_start),
                                       _p(slot), _p(state), _p(scratch), _p(scratch[B * H * nc:]), _p(out),
                                       out.stride(0), chunk, nc, _stream()), "decay_chunked")
        add_launches(2)
        return
    _check(load().kb_decay_scan(_p(a), dt(a), n_planes, pstride, ld, B, H, d, dv, _p(decay), _p(q_start), _p(slot),
                                _p(state), _p(out), out.stride(0), _stream()), "decay_scan")


MOE_SCORE = {"softmax": 0, "sigmoid": 1}


def moe_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], top: int, score: str = "softmax",
             n_experts: Optional[int] = None):
    """the ``top`` largest of each row of logits + bias (float32 [T, >= E]; ``n_experts``: the first E columns are
    the experts') and their weights: the softmax over those alone (``score`` "softmax") or each one's own sigmoid, not
    normalised ("sigmoid"): (idx int32 [T, top], weights float32 [T, top])"""
    _need_cuda(logits, bias)
    T, E = logits.shape
    if n_experts is not None:
        assert n_experts <= E
        E = n_experts
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == E and bias.is_contiguous()
    if not (1 <= top <= min(E, 32)):
        raise KernelError("kindi_b200: a row picks 1 to 32 of its %d experts, found top = %d" % (E, top))
    idx = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    wts = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    _check(load().kb_moe_topk(_p(logits), logits.stride(0), _p(bias), T, E, top, _p(idx), _p(wts), _stream(),
                              MOE_SCORE[score]), "moe_topk")
    return idx, wts


class MoePlan:
    """(row, pick) pairs sorted by expert and cut into tiles, all on the device (see ``csrc/moe.cu``)"""

    __slots__ = ("n_pairs", "n_experts", "tile", "max_tiles", "offs", "perm", "tile_e", "tile_r0", "n_tiles")


def _new_plan(n: int, n_experts: int, tile: int, device) -> MoePlan:
    pl = MoePlan()
    pl.n_pairs, pl.n_experts, pl.tile = n, n_experts, tile
    pl.max_tiles = -(-n // tile) + min(n_experts, n)
    buf = torch.empty(n_experts + 1 + n + 2 * pl.max_tiles + 1, dtype=torch.int32, device=device)
    a = 0
    pl.offs = buf[a:a + n_experts + 1]
    a += n_experts + 1
    pl.perm = buf[a:a + n]
    a += n
    pl.tile_e = buf[a:a + pl.max_tiles]
    a += pl.max_tiles
    pl.tile_r0 = buf[a:a + pl.max_tiles]
    a += pl.max_tiles
    pl.n_tiles = buf[a:a + 1]
    return pl


def moe_plan(idx: torch.Tensor, n_experts: int, tile: int) -> MoePlan:
    _need_cuda(idx)
    assert idx.dtype == torch.int32 and idx.is_contiguous()
    n = idx.numel()
    if n_experts > 4096:
        raise KernelError("kindi_b200: up to 4096 experts, found %d" % n_experts)
    pl = _new_plan(n, n_experts, tile, idx.device)
    _check(load().kb_moe_plan(_p(idx), n, n_experts, tile, _p(pl.offs), _p(pl.perm), _p(pl.tile_e), _p(pl.tile_r0),
                              _p(pl.n_tiles), _stream()), "moe_plan")
    return pl


@functools.lru_cache(maxsize=1)
def moe_gemm_tile() -> int:
    return load().kb_moe_gemm_tile()


def moe_gemm_up(y: torch.Tensor, w: torch.Tensor, plan: MoePlan, top: int, act: str, out: torch.Tensor) -> None:
    """out[r] (sorted rows [n_pairs, F]) = act(y[token of pair perm[r]] @ w[expert of r]^T); w [E, F, K]"""
    _need_cuda(y, w, out)
    E, F, Kd = w.shape
    assert y.stride(1) == 1 and y.shape[1] == Kd and w.is_contiguous() and out.shape == (plan.n_pairs, F)
    assert out.stride(1) == 1 and plan.tile == moe_gemm_tile()
    _check(load().kb_moe_gemm(_p(y), dt(y), y.stride(0), _p(w), dt(w), _p(out), dt(out), out.stride(0), 0, F, Kd,
                              plan.max_tiles, _p(plan.n_tiles), _p(plan.tile_e), _p(plan.tile_r0), _p(plan.offs),
                              _p(plan.perm), None, top, ACT[act], 1, _stream()), "moe_gemm_up")


def moe_gemm_down(h: torch.Tensor, w: torch.Tensor, plan: MoePlan, wts: torch.Tensor, top: int,
                  planes: torch.Tensor) -> None:
    """planes[k][t] (float32 [top, T, N]) = wts[t][k] * (h[sorted row of pair (t, k)] @ w[its expert]^T); w [E, N, F]"""
    _need_cuda(h, w, planes, wts)
    E, N, F = w.shape
    assert h.stride(1) == 1 and h.shape == (plan.n_pairs, F) and w.is_contiguous()
    assert planes.dtype == torch.float32 and planes.is_contiguous() and planes.shape[0] == top and planes.shape[2] == N
    assert wts.dtype == torch.float32 and wts.is_contiguous() and wts.numel() == plan.n_pairs
    _check(load().kb_moe_gemm(_p(h), dt(h), h.stride(0), _p(w), dt(w), _p(planes), F32, N,
                              planes.stride(0), N, F, plan.max_tiles, _p(plan.n_tiles), _p(plan.tile_e),
                              _p(plan.tile_r0), _p(plan.offs), _p(plan.perm), _p(wts), top, 0, 0, _stream()),
           "moe_gemm_down")


@functools.lru_cache(maxsize=1)
def moe_gemm_tc_tile() -> int:
    return load().kb_moe_gemm_tc_tile()


def moe_gather(y: torch.Tensor, out: torch.Tensor, plan: MoePlan, top: int) -> None:
    """out[r] = y[token of pair perm[r]]: the activation rows in the plan's order (bf16, width a multiple of 8)"""
    _need_cuda(y, out)
    assert y.dtype == out.dtype == torch.bfloat16 and y.stride(1) == 1 and out.is_contiguous()
    assert out.shape == (plan.n_pairs, y.shape[1])
    _check(load().kb_moe_gather(_p(y), y.stride(0), _p(out), y.shape[1], _p(plan.perm), plan.n_pairs, top, _stream()),
           "moe_gather")


def moe_gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, plan: MoePlan, wts: Optional[torch.Tensor],
                top: int, act: str, *, up: bool, bn: int, status: torch.Tensor, glu: bool = False,
                act_params=None) -> None:
    """the experts' grouped product on the tensor cores over the plan's tiles of 128 sorted rows. a: sorted rows
    [n_pairs, K] bf16; w [E, N, K] bf16. up: out = act(a w[e]^T) as bf16 [n_pairs, N]; else out = float planes
    [top, T, N] with plane k of a row's token = its k-th weight * (a w[e]^T). ``glu`` (up form): every expert's rows
    are 16 gate rows then the 16 up rows of the same outputs, group after group, ``act`` names the gated unit (a key of
    ``GATE_ACT``, with ``act_params``) and out [n_pairs, N / 2] holds the finished unit"""
    _need_cuda(a, w, out, wts)
    E, N, Kd = w.shape
    assert a.dtype == w.dtype == torch.bfloat16 and a.shape == (plan.n_pairs, Kd) and a.stride(1) == 1
    assert w.is_contiguous() and plan.tile == moe_gemm_tc_tile() and bn in (64, 128, 256)
    if up:
        n_out = N // 2 if glu else N
        assert not glu or N % 32 == 0
        assert out.dtype == torch.bfloat16 and out.shape == (plan.n_pairs, n_out) and out.stride(1) == 1
        ldc, pstride = out.stride(0), 0
    else:
        assert out.dtype == torch.float32 and out.is_contiguous() and out.shape[0] == top and out.shape[2] == N
        assert wts is not None and wts.dtype == torch.float32 and wts.is_contiguous() and wts.numel() == plan.n_pairs
        ldc, pstride = N, out.stride(0)
    _check(load().kb_moe_gemm_tc(_p(a), plan.n_pairs, a.stride(0), _p(w), E, N, Kd, _p(out), ldc, pstride,
                                 plan.max_tiles, _p(plan.n_tiles), _p(plan.tile_e), _p(plan.tile_r0), _p(plan.offs),
                                 _p(plan.perm), _p(wts), top, GATE_ACT[act] if glu else ACT[act], 1 if up else 0, bn,
                                 _p(status), _stream(), 1 if glu else 0, *_gate_params(act if glu else "", act_params)),
           "moe_gemm_tc")


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T with 32-bit accumulation in a fixed order (no tensor cores)"""
    _need_cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(load().kb_gemm_simt(_p(a), dt(a), _p(w), dt(w), _p(out), dt(out), M, N, K, a.stride(0), w.stride(0),
                               out.stride(0), _stream()), "gemm_simt")


@functools.lru_cache(maxsize=1)
def rope_table_min_rows() -> int:
    """steps of fewer rows are rotated by kernels that compute their angles themselves and read no table"""
    return load().kb_rope_table_min_rows()


def rope_table(pos: torch.Tensor, inv_freq: torch.Tensor, rot: int) -> torch.Tensor:
    """(cos, sin) of float(pos[t]) * inv_freq[i] for every row and rotated pair: float32 [T, rot / 2, 2]. The angles of
    a step are the same in every layer, so a step makes this once and hands it to ``rope_store``"""
    _need_cuda(pos, inv_freq)
    T = pos.numel()
    assert pos.dtype == torch.int32 and inv_freq.dtype == torch.float32 and rot % 2 == 0
    assert inv_freq.numel() >= max(1, rot // 2)
    out = torch.empty((T, rot // 2, 2), dtype=torch.float32, device=pos.device)
    _check(load().kb_rope_table(_p(pos), _p(inv_freq), rot, T, _p(out), _stream()), "rope_table")
    return out


def rope_store(qkv: torch.Tensor, qout: torch.Tensor, inv_freq: torch.Tensor, rot: int, pos, seq, slot, nh: int,
               nkv: int, hd: int, pool: Optional[torch.Tensor], table: torch.Tensor, n_pages: int,
               status: torch.Tensor, angles: Optional[torch.Tensor] = None) -> None:
    """qkv: [T, (nh + 2 nkv) hd], or 32-bit planes [S, T, ...] that are summed. Query heads are rotated into qout
    ([T, >= nh hd]; may be qkv itself), keys are rotated and stored in the cache, values are stored. ``angles``: what
    ``rope_table`` made for these rows (optional: without it the kernel computes the cosines and sines itself)"""
    _need_cuda(qkv, qout, inv_freq, pool, table)
    planes = qkv.shape[0] if qkv.dim() == 3 else 1
    T = qkv.shape[-2]
    assert qkv.stride(-1) == 1 and inv_freq.dtype == torch.float32 and inv_freq.numel() >= max(1, rot // 2)
    assert rot % 2 == 0 and rot <= hd and qout.stride(1) == 1
    if pool is not None:
        assert pool.dtype == qout.dtype and pool.is_contiguous()
    pstride = qkv.stride(0) if qkv.dim() == 3 else 0
    if angles is not None:
        assert angles.dtype == torch.float32 and angles.is_contiguous() and angles.shape == (T, rot // 2, 2)
    _check(load().kb_rope_store(_p(qkv), dt(qkv), planes, pstride, qkv.stride(-2), _p(qout), dt(qout),
                                qout.stride(0), _p(inv_freq), rot, _p(pos), _p(seq), _p(slot), T, nh, nkv, hd,
                                _p(pool), _p(table), table.stride(0), n_pages, _p(status), _stream(), _p(angles)),
           "rope_store")


def attn_generic(q: torch.Tensor, out: torch.Tensor, pos, seq, slot, nh: int, nkv: int, hd: int, scale: float,
                 window: int, pool: torch.Tensor, table: torch.Tensor, n_pages: int, status: torch.Tensor,
                 keep_first: int = 0, sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None) -> None:
    """attention of each row of q ([T, >= nh hd], row stride free) over its sequence's cached keys and values: all
    positions up to the row's, or with ``window`` the last ``window`` of them and the sequence's first ``keep_first``.
    ``sink`` (float32 [nh]): exp(sink[h]) joins head h's softmax denominator. ``gate`` (rows of q's dtype, laid out
    like ``out``): the output is multiplied by the logistic function of it"""
    _need_cuda(q, out, pool, table, sink, gate)
    if sink is not None:
        assert sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == nh
    if gate is not None:
        assert gate.dtype == q.dtype and gate.stride(1) == 1 and gate.shape[0] == q.shape[0]
    T = q.shape[0]
    if hd > 512:
        raise KernelError("kindi_b200: attention supports head sizes up to 512, found %d" % hd)
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == pool.dtype
    _check(load().kb_attn_generic(_p(q), dt(q), q.stride(0), _p(out), out.stride(0), _p(pos), _p(seq), _p(slot), T,
                                  nh, nkv, hd, float(scale), int(window), _p(pool), _p(table), table.stride(0),
                                  n_pages, _p(status), _stream(), int(keep_first), _p(sink), _p(gate),
                                  gate.stride(0) if gate is not None else 0), "attn_generic")


def swiglu(gu: torch.Tensor, out: torch.Tensor, group: int = 0, act: str = "silu") -> None:
    """out[T, F] = act(g) * u with gu [T, 2F] (or the sum of 32-bit planes gu [S, T, 2F]). The columns of gu come in
    groups of ``group`` gate columns followed by the ``group`` up columns of the same outputs (0: all gates, then
    all ups). ``act``: "silu" or "gelu_tanh"."""
    _need_cuda(gu, out)
    T, F = out.shape
    planes = gu.shape[0] if gu.dim() == 3 else 1
    assert gu.shape[-2:] == (T, 2 * F) and gu.is_contiguous() and out.is_contiguous()
    _check(load().kb_swiglu(_p(gu), dt(gu), planes, T * 2 * F, _p(out), dt(out), T, F, group or F, _stream(),
                            GATE_ACT[act]), "swiglu")


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, swap: bool, bn: int, splits: int,
            status: torch.Tensor, swiglu: bool = False, mt: int = 1, act: str = "silu", act_params=None) -> None:
    """out = a[M, K] @ w[N, K]^T on the tensor cores (bf16 in, fp32 accumulate). ``out`` is [M, N] (bf16 or fp32)
    or, with K splits, fp32 [S, M, N] where S = gemm_tc_splits(K, splits). ``swiglu`` (prefill form, bn a multiple
    of 32): w holds 16 gate rows then the 16 up rows of the same outputs, group after group, and ``out`` is the bf16
    [M, N / 2] result silu(gate) * up. ``mt`` = 2 (prefill form): a unit is two 128-row tiles over the same columns"""
    _need_cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.is_contiguous()
    if swiglu:
        assert out.shape == (M, N // 2) and out.dtype == torch.bfloat16 and not swap and splits == 1 and N % 32 == 0 and bn % 32 == 0
        stride, ldc = 0, N // 2
    elif out.dim() == 3:
        assert out.shape == (gemm_tc_splits(K, splits), M, N) and out.dtype == torch.float32
        stride, ldc = M * N, N
    else:
        assert out.shape == (M, N) and splits == 1
        stride, ldc = 0, N
    _check(load().kb_gemm_tc(_p(a), _p(w), _p(out), dt(out), M, N, K, a.stride(0), w.stride(0), ldc, 1 if swap else 0,
                             bn, splits, stride, _p(status), _stream(), GATE_ACT[act] if swiglu else 0, mt,
                             *_gate_params(act, act_params)), "gemm_tc")


def gemm_pair(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bn: int, status: torch.Tensor,
              swiglu: bool = False, part: Optional[torch.Tensor] = None, flags: Optional[torch.Tensor] = None,
              act: str = "silu", act_params=None) -> None:
    """out = a[M, K] @ w[N, K]^T by pairs of SMs (tcgen05 with cta_group::2: a pair computes 256 rows x bn columns,
    each CTA holding half of the weight tile), bf16 in, fp32 accumulate, ``out`` [M, N] bf16 or fp32; bn 64, 128, 192
    or 256. ``swiglu``: as for gemm_tc, ``out`` is the bf16 [M, N / 2] result silu(gate) * up. With ``part`` (fp32, at
    least tiles * 256 * bn elements, tiles = ceil(M / 256) * ceil(N / bn)) and ``flags`` (int32 zeros, 8 a tile) the
    K blocks of all tiles are dealt out evenly to the pairs and a tile may be finished by two of them"""
    _need_cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.is_contiguous() and bn in (64, 128, 192, 256)
    if swiglu:
        assert out.shape == (M, N // 2) and out.dtype == torch.bfloat16 and N % 32 == 0
        ldc = N // 2
    else:
        assert out.shape == (M, N)
        ldc = N
    if part is not None:
        tiles = -(-M // 256) * -(-N // bn)
        assert part.dtype == torch.float32 and part.numel() >= tiles * 256 * bn and part.is_contiguous()
        assert flags.dtype == torch.int32 and flags.numel() >= 8 * tiles and flags.is_contiguous()
    _check(load().kb_gemm_pair(_p(a), _p(w), _p(out), dt(out), M, N, K, a.stride(0), w.stride(0), ldc, bn, _p(status),
                               _stream(), GATE_ACT[act] if swiglu else 0, _p(part), _p(flags),
                               *_gate_params(act, act_params)), "gemm_pair")


def gemm_swiglu_decode(a: torch.Tensor, w_grouped: torch.Tensor, out: torch.Tensor, bn: int, part: torch.Tensor,
                       flags: torch.Tensor, status: torch.Tensor, act: str = "silu", act_params=None) -> None:
    """out (bf16 [M, F]) = silu(g) * u with [g | u] = a[M, K] @ w_grouped[2F, K]^T (16 gate rows, then the 16 up rows
    of the same outputs), for M <= bn rows, SwiGLU finished inside the product. ``part`` (float32, at least
    ceil(2F / 128) * bn * 128) and ``flags`` (int32 zeros, at least ceil(2F / 128)) are scratch that calls on one
    stream may share"""
    _need_cuda(a, w_grouped, out, part, flags)
    M, K = a.shape
    F = w_grouped.shape[0] // 2
    tiles = -(-2 * F // 128)
    assert a.dtype == w_grouped.dtype == out.dtype == torch.bfloat16 and w_grouped.shape == (2 * F, K)
    assert a.stride(1) == 1 and w_grouped.stride(1) == 1 and out.shape == (M, F) and out.stride(1) == 1
    assert F % 16 == 0 and M <= bn and part.dtype == torch.float32 and part.numel() >= tiles * bn * 128
    assert flags.dtype == torch.int32 and flags.numel() >= tiles
    _check(load().kb_gemm_swiglu_decode(_p(a), _p(w_grouped), _p(out), M, F, K, a.stride(0), w_grouped.stride(0),
                                        out.stride(0), bn, _p(part), _p(flags), _p(status), _stream(), GATE_ACT[act],
                                        *_gate_params(act, act_params)), "gemm_swiglu_decode")


@functools.lru_cache(maxsize=4096)
def gemm_tc_splits(K: int, wanted: int) -> int:
    return load().kb_gemm_tc_splits(K, wanted)


def attn_mma(q: torch.Tensor, out: torch.Tensor, slot, q_start, kv_len, B: int, nh: int, nkv: int, hd: int,
             scale: float, window: int, pool: torch.Tensor, table: torch.Tensor, n_pages: int, *, decode: bool,
             grid_x: int, status: torch.Tensor, keep_first: int = 0, sink: Optional[torch.Tensor] = None) -> None:
    """tensor-core attention over the cache (bf16, head size 64 or 128). decode: one row per sequence, grid_x =
    position splits; else grid_x = ceil(most rows of a sequence * (nh / nkv) / 64). ``keep_first``: with a window,
    the sequence's first positions that stay visible. ``sink`` (float32 [nh]): exp(sink[h]) joins head h's softmax
    denominator"""
    _need_cuda(q, out, pool, table, sink)
    if sink is not None:
        assert sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == nh
    assert q.dtype == out.dtype == pool.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert pool.is_contiguous()
    part_o = part_ml = None
    if decode and grid_x > 1:
        part_o = torch.empty((B, nh, grid_x, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((B, nh, grid_x, 2), dtype=torch.float32, device=q.device)
    _check(load().kb_attn_mma(_p(q), q.stride(0), _p(out), out.stride(0), _p(part_o), _p(part_ml), _p(slot),
                              _p(q_start), _p(kv_len), B, nh, nkv, hd, float(scale), int(window), _p(pool), _p(table),
                              table.stride(0), n_pages, 1 if decode else 0, grid_x, _p(status), _stream(),
                              int(keep_first), _p(sink)), "attn_mma")
    if decode and grid_x > 1:
        add_launches(1)         # the merge of the position splits


def attn_decode_rope(qkv: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor, slot, q_start, kv_len, B: int,
                     nh: int, nkv: int, hd: int, scale: float, window: int, pool: torch.Tensor, store: bool,
                     table: torch.Tensor, n_pages: int, *, grid_x: int, status: torch.Tensor) -> None:
    """decode attention that takes the QKV product as 32-bit planes [S, rows, (nh + 2 nkv) hd], rotates the queries
    and the newest key over the whole head, stores the newest key and value (``store``) and attends; grid_x =
    position splits"""
    _need_cuda(qkv, out, pool, table, inv_freq)
    assert qkv.dtype == torch.float32 and qkv.dim() == 3 and qkv.stride(2) == 1 and qkv.stride(1) == qkv.shape[2]
    assert out.dtype == pool.dtype == torch.bfloat16 and out.stride(1) == 1 and pool.is_contiguous()
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == hd // 2
    part_o = part_ml = None
    if grid_x > 1:
        part_o = torch.empty((B, nh, grid_x, hd), dtype=torch.float32, device=out.device)
        part_ml = torch.empty((B, nh, grid_x, 2), dtype=torch.float32, device=out.device)
    _check(load().kb_attn_decode_rope(_p(qkv), qkv.shape[0], qkv.stride(0), qkv.stride(1), _p(inv_freq), _p(out),
                                      out.stride(0), _p(part_o), _p(part_ml), _p(slot), _p(q_start), _p(kv_len), B, nh,
                                      nkv, hd, float(scale), int(window), _p(pool), 1 if store else 0, _p(table),
                                      table.stride(0), n_pages, grid_x, _p(status), _stream()), "attn_decode_rope")
    if grid_x > 1:
        add_launches(1)         # the merge of the position splits


def attn_tc(q: torch.Tensor, out: torch.Tensor, slot, q_start, kv_len, B: int, nh: int, nkv: int, hd: int,
            scale: float, window: int, pool: torch.Tensor, table: torch.Tensor, n_pages: int, *, grid_x: int,
            status: torch.Tensor, keep_first: int = 0, sink: Optional[torch.Tensor] = None,
            gate: Optional[torch.Tensor] = None) -> None:
    """tcgen05 attention for prompt-sized steps (bf16, head size 64 or 128): grid_x = ceil(most rows of a sequence /
    (128 // (nh / nkv))). ``keep_first``: with a window, the sequence's first positions that stay visible. ``sink``
    (float32 [nh]): exp(sink[h]) joins head h's softmax denominator. ``gate`` (bf16 rows laid out like ``out``, rows
    16-byte aligned): the output is multiplied by the logistic function of it"""
    _need_cuda(q, out, pool, table, sink, gate)
    if sink is not None:
        assert sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == nh
    if gate is not None:
        assert gate.dtype == torch.bfloat16 and gate.stride(1) == 1 and gate.shape[0] == q.shape[0]
    assert q.dtype == out.dtype == pool.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert pool.is_contiguous() and hd in (64, 128)
    _check(load().kb_attn_tc(_p(q), q.stride(0), _p(out), out.stride(0), _p(slot), _p(q_start), _p(kv_len), B, nh, nkv,
                             hd, float(scale), int(window), _p(pool), _p(table), table.stride(0), n_pages, grid_x,
                             _p(status), _stream(), int(keep_first), _p(sink), _p(gate),
                             gate.stride(0) if gate is not None else 0), "attn_tc")


# ----------------------------------------------------------------------------------------------- stateful mixers
GATE_KIND = {"none": 0, "sigmoid": 1, "silu": 2}


def sinusoid_add(x: torch.Tensor, pos: torch.Tensor, freq: torch.Tensor) -> None:
    """x[t][2i] += sin(pos[t] * freq[i]), x[t][2i + 1] += cos(pos[t] * freq[i]); x float32 [T, E], freq float64"""
    _need_cuda(x, pos, freq)
    T, E = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and freq.dtype == torch.float64 and freq.is_contiguous()
    assert freq.numel() >= (E + 1) // 2 and pos.dtype == torch.int32
    _check(load().kb_sinusoid_add(_p(x), _p(pos), _p(freq), T, E, _stream()), "sinusoid_add")


def mix_cat(x: torch.Tensor, delta: Optional[torch.Tensor], scale: Optional[torch.Tensor], x0: torch.Tensor,
            out: torch.Tensor) -> None:
    """out[t] = [x[t] + scale * (sum of delta's planes)[t] | x0[t]]; x, x0 float32 [T, E], out [T, 2 E]"""
    _need_cuda(x, delta, scale, x0, out)
    T, E = x.shape
    assert x.dtype == x0.dtype == torch.float32 and x.is_contiguous() and x0.is_contiguous() and x0.shape == x.shape
    assert out.is_contiguous() and out.shape == (T, 2 * E)
    nd, stride = 0, 0
    if delta is not None:
        assert delta.dtype == torch.float32 and delta.is_contiguous() and delta.shape[1:] == (T, E)
        nd, stride = delta.shape[0], T * E
    if scale is not None:
        assert scale.dtype == torch.float32 and scale.is_contiguous() and scale.numel() == E
    _check(load().kb_mix_cat(_p(x), _p(delta), nd, stride, _p(scale) if delta is not None else None, _p(x0), _p(out),
                             dt(out), T, E, _stream()), "mix_cat")


def short_conv(a: torch.Tensor, col0: int, C: int, bias: Optional[torch.Tensor], w: torch.Tensor, act: bool,
               tails: torch.Tensor, pos, seq, slot, q_start, out: torch.Tensor) -> None:
    """causal convolution over time per channel on columns ``col0 .. col0 + C`` of ``a`` (rows or 32-bit planes), plus
    ``bias`` before the convolution; ``w`` float32 [C, taps] (the last tap meets the current token); ``act``: silu
    after it. ``tails``: float32 [slots, >= (taps - 1) * C] (a view whose rows may be strided), the sequence's last
    taps - 1 inputs, read for positions before this step and rewritten. ``out`` [T, C] (a view is fine)"""
    _need_cuda(a, bias, w, tails, out)
    n_planes, pstride, ld = _planes_of(a)
    T = a.shape[-2]
    taps = w.shape[1]
    assert w.dtype == torch.float32 and w.is_contiguous() and w.shape[0] == C and a.shape[-1] >= col0 + C
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == C)
    assert tails.dtype == torch.float32 and tails.stride(1) == 1 and tails.shape[1] >= (taps - 1) * C
    assert out.shape == (T, C) and out.stride(1) == 1
    if not (1 <= taps <= 8):
        raise KernelError("kindi_b200: a short convolution has 1 to 8 taps, found %d" % taps)
    _check(load().kb_short_conv(_p(a), dt(a), n_planes, pstride, ld, col0, C, _p(bias), _p(w), taps, 1 if act else 0,
                                _p(tails), tails.stride(0), _p(pos), _p(seq), _p(slot), _p(q_start), _p(out), dt(out),
                                out.stride(0), T, _stream()), "short_conv")


DELTA_CHUNK = 64            # rows of a run (DC_C of the kernels)
DELTA_CHUNKED = 128         # sequences that bring more rows than this run in the chunked form


def delta_rule(qkv: torch.Tensor, proj: torch.Tensor, ob: int, oa: int, a_log: torch.Tensor, dt_bias: torch.Tensor,
               B: int, H: int, G: int, d: int, dv: int, unit_eps: float, q_start, slot, state: torch.Tensor,
               out: torch.Tensor, max_rows: int = 0) -> None:
    """the gated delta rule over the packed rows of ``B`` sequences. ``qkv`` float32 rows [q (G d) | k (G d) | v (H dv)];
    ``proj`` (rows or 32-bit planes) holds the beta logits at columns ``ob ..`` and the decay's at ``oa ..`` (H each);
    ``state`` float32 [slots, >= H dv d] (rows may be strided) is read and written; ``out`` float32 [T, H dv].
    ``max_rows`` (the most rows a sequence brings, or an upper bound) above ``DELTA_CHUNKED`` selects the form for long
    prompts, which works a sequence in runs of ``DELTA_CHUNK`` rows (per run a triangular system that does not depend
    on the state, solved for all runs side by side, then five small products a run); its sums differ from the
    token-by-token form's by rounding"""
    _need_cuda(qkv, proj, a_log, dt_bias, state, out)
    n_planes, pstride, ldp = _planes_of(proj)
    assert qkv.dtype == torch.float32 and qkv.stride(1) == 1 and qkv.shape[1] >= 2 * G * d + H * dv
    assert a_log.dtype == dt_bias.dtype == torch.float32 and a_log.numel() == H == dt_bias.numel()
    assert state.dtype == torch.float32 and state.stride(1) == 1 and state.shape[1] >= H * dv * d
    assert out.dtype == torch.float32 and out.stride(1) == 1 and out.shape[1] == H * dv
    if d > 256:
        raise KernelError("kindi_b200: the delta rule supports key sizes up to 256, found %d" % d)
    if max_rows > DELTA_CHUNKED:
        lib = load()
        nc = -(-int(max_rows) // DELTA_CHUNK)
        # per (sequence, run, head) the solved system, the weights of the run's own keys and three vectors; per
        # (sequence, run, key head) the unit keys and queries, rows padded to a multiple of four
        C, dp = DELTA_CHUNK, (d + 3) // 4 * 4
        hs = torch.empty(B * nc * H * (2 * C * C + 3 * C), dtype=torch.float32, device=out.device)
        qk = torch.empty(B * nc * G * 2 * C * dp, dtype=torch.float32, device=out.device)
        _check(lib.kb_delta_chunked(_p(qkv), qkv.stride(0), _p(proj), dt(proj), n_planes, pstride, ldp, ob, oa,
                                    _p(a_log), _p(dt_bias), B, H, G, d, dv, float(unit_eps), _p(q_start), _p(slot),
                                    _p(state), state.stride(0), _p(hs), _p(qk), nc, _p(out), out.stride(0), _stream()),
               "delta_chunked")
        add_launches(1)
        return
    _check(load().kb_delta_rule(_p(qkv), qkv.stride(0), _p(proj), dt(proj), n_planes, pstride, ldp, ob, oa, _p(a_log),
                                _p(dt_bias), B, H, G, d, dv, float(unit_eps), _p(q_start), _p(slot), _p(state),
                                state.stride(0), _p(out), out.stride(0), _stream()), "delta_rule")


def head_norm_gate(x: torch.Tensor, H: int, n: int, w: torch.Tensor, eps: float, g: Optional[torch.Tensor], og: int,
                   gate: str, out: torch.Tensor) -> None:
    """out[t][h n + e] = x[t][h n + e] / sqrt(mean_e x^2 + eps) * w[e] * gate(g[t][og + h n + e]); x float32 [T, H n],
    w float32 [n], ``g`` rows or 32-bit planes, ``gate``: none, sigmoid or silu"""
    _need_cuda(x, w, g, out)
    T = x.shape[0]
    assert x.dtype == torch.float32 and x.stride(1) == 1 and x.shape[1] == H * n and w.dtype == torch.float32
    assert w.numel() == n and w.is_contiguous() and out.shape == (T, H * n) and out.stride(1) == 1
    n_planes, pstride, ldg = _planes_of(g) if g is not None else (1, 0, 0)
    _check(load().kb_head_norm_gate(_p(x), x.stride(0), T, H, n, _p(w), float(eps), _p(g),
                                    dt(g) if g is not None else F32, n_planes, pstride, ldg, og, GATE_KIND[gate],
                                    _p(out), dt(out), out.stride(0), _stream()), "head_norm_gate")


MIN_GRU_CHUNK = 64          # rows of a chunk (MG_CHUNK of the kernel)
MIN_GRU_CHUNKED = 128       # sequences that bring more rows than this run in chunks


def min_gru(a: torch.Tensor, oz: int, ox: int, og: int, W: int, bz: Optional[torch.Tensor],
            bx: Optional[torch.Tensor], B: int, q_start, slot, state: torch.Tensor, out: torch.Tensor,
            max_rows: int = 0) -> None:
    """S <- (1 - z) S + z c per element over the packed rows of ``B`` sequences: z = sigmoid(a[oz ..] + bz),
    u = a[ox ..] + bx, c = u + 1/2 where u >= 0 else sigmoid(u); out = S * silu(a[og ..]). ``state`` float32
    [slots, >= W] (rows may be strided). ``max_rows`` (the most rows a sequence brings, or an upper bound) above
    ``MIN_GRU_CHUNKED`` selects the form for long prompts, which works on a sequence's runs of ``MIN_GRU_CHUNK`` rows
    side by side; its states differ from the token-by-token form's by rounding"""
    _need_cuda(a, bz, bx, state, out)
    n_planes, pstride, ld = _planes_of(a)
    T = a.shape[-2]
    for b_ in (bz, bx):
        assert b_ is None or (b_.dtype == torch.float32 and b_.is_contiguous() and b_.numel() == W)
    assert state.dtype == torch.float32 and state.stride(1) == 1 and state.shape[1] >= W
    assert out.shape == (T, W) and out.stride(1) == 1
    nc, part = 0, None
    if max_rows > MIN_GRU_CHUNKED:
        nc = -(-int(max_rows) // MIN_GRU_CHUNK)
        part = torch.empty((B, nc, 2, W), dtype=torch.float32, device=out.device)
        add_launches(1)
    _check(load().kb_min_gru(_p(a), dt(a), n_planes, pstride, ld, oz, ox, og, W, _p(bz), _p(bx), B, _p(q_start),
                             _p(slot), _p(state), state.stride(0), _p(out), dt(out), out.stride(0), _p(part), nc,
                             _stream()), "min_gru")


def branch_norm_mean(branches, eps: float, out: torch.Tensor) -> None:
    """out (float32 [T, E]) = the mean over ``branches`` of rms(sum of planes + bias) * gain; each branch is
    ``(planes float32 [S, T, E], bias float32 [E] or None, gain float32 [E])``, at most four"""
    n = len(branches)
    T, E = out.shape
    assert 1 <= n <= 4 and out.dtype == torch.float32 and out.is_contiguous()
    ptrs, counts, strides, biases, gains = [], [], [], [], []
    for planes, bias, gain in branches:
        _need_cuda(planes, bias, gain)
        assert planes.dtype == torch.float32 and planes.is_contiguous() and planes.shape[1:] == (T, E)
        assert gain.dtype == torch.float32 and gain.is_contiguous() and gain.numel() == E
        assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == E)
        ptrs.append(_p(planes))
        counts.append(planes.shape[0])
        strides.append(T * E)
        biases.append(_p(bias))
        gains.append(_p(gain))
    arr = (c_void_p * n)
    _check(load().kb_branch_norm_mean(n, arr(*ptrs), (c_int * n)(*counts), (c_longlong * n)(*strides), arr(*biases),
                                      arr(*gains), float(eps), _p(out), T, E, _stream()), "branch_norm_mean")


def moe_gate_mul(gu: torch.Tensor, wts: Optional[torch.Tensor], plan: "MoePlan", act: str, h: torch.Tensor) -> None:
    """h[r] = act(w g) * (w u) over the plan's sorted rows: ``gu`` [n_pairs, 2 F] = [gate | up], w = the weight of the
    row's (token, pick) pair"""
    _need_cuda(gu, wts, h)
    n, F2 = gu.shape
    F = F2 // 2
    assert gu.stride(1) == 1 and h.shape == (n, F) and h.stride(1) == 1 and h.dtype == gu.dtype and n == plan.n_pairs
    assert wts is None or (wts.dtype == torch.float32 and wts.is_contiguous() and wts.numel() == n)
    _check(load().kb_moe_gate_mul(_p(gu), dt(gu), gu.stride(0), _p(wts), _p(plan.perm), n, F, ACT[act], _p(h),
                                  h.stride(0), _stream()), "moe_gate_mul")


def row_gate(h: torch.Tensor, z: torch.Tensor) -> None:
    """h[t] *= sigmoid(z[t]); ``z`` float32 [T] (a strided view is fine); in place"""
    _need_cuda(h, z)
    T, N = h.shape
    assert h.stride(1) == 1 and z.dtype == torch.float32 and z.numel() == T and z.dim() == 1
    _check(load().kb_row_gate(_p(h), dt(h), h.stride(0), _p(z), z.stride(0), T, N, _stream()), "row_gate")


def sigattn_prep(c: torch.Tensor, H: int, G: int, d: int, dv: int, hd: int, coef: float, every: int, v_norm: bool,
                 eps: float, pos, seq, slot, q_out: torch.Tensor, pool: torch.Tensor, table: torch.Tensor, n_pages: int,
                 status: torch.Tensor) -> None:
    """``c`` float32 rows [q (H d) | k (G d) | v (G dv)]: queries times ``1 + coef ln((pos + 1) // every + 1)`` to
    ``q_out`` [T, H hd]; keys, and values divided per head by their root mean square (``v_norm``), into the cache"""
    _need_cuda(c, q_out, pool, table)
    T = c.shape[0]
    assert c.dtype == torch.float32 and c.stride(1) == 1 and c.shape[1] >= H * d + G * d + G * dv
    assert q_out.shape == (T, H * hd) and q_out.stride(1) == 1 and pool.dtype == q_out.dtype and pool.is_contiguous()
    assert pool.shape[-1] == hd and pool.shape[-3] == G
    _check(load().kb_sigattn_prep(_p(c), c.stride(0), T, H, G, d, dv, hd, float(coef), int(every), 1 if v_norm else 0,
                                  float(eps), _p(pos), _p(seq), _p(slot), _p(q_out), dt(q_out), q_out.stride(0),
                                  _p(pool), _p(table), table.stride(0), n_pages, _p(status), _stream()), "sigattn_prep")


def sigmoid_attn(q: torch.Tensor, out: torch.Tensor, pos, seq, slot, nh: int, nkv: int, hd: int, scale: float,
                 bias: Optional[torch.Tensor], pool: torch.Tensor, table: torch.Tensor, n_pages: int,
                 status: torch.Tensor) -> None:
    """causal attention whose weights are sigmoid(q . k * scale + bias[h][distance]) without normalisation (the
    general kernel); ``bias`` float32 [nh, n] over the distance, its last entry for every larger distance, or None"""
    _need_cuda(q, out, bias, pool, table)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == pool.dtype and pool.is_contiguous()
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.shape[0] == nh)
    if hd > 512:
        raise KernelError("kindi_b200: head sizes up to 512 are supported, found %d" % hd)
    _check(load().kb_sigmoid_attn(_p(q), dt(q), q.stride(0), _p(out), out.stride(0), _p(pos), _p(seq), _p(slot), T, nh,
                                  nkv, hd, float(scale), _p(bias), bias.shape[1] if bias is not None else 0, _p(pool),
                                  _p(table), table.stride(0), n_pages, _p(status), _stream()), "sigmoid_attn")


def sigattn_decode(q: torch.Tensor, out: torch.Tensor, slot, kv_len, B: int, nh: int, nkv: int, hd: int, scale: float,
                   bias: Optional[torch.Tensor], pool: torch.Tensor, table: torch.Tensor, n_pages: int, *, splits: int,
                   status: torch.Tensor) -> None:
    """attention without a softmax for single tokens (float32 or bf16 storage, 32-bit arithmetic): row b of ``q`` and
    ``out`` is sequence b's newest position ``kv_len[b] - 1``; every sequence's pages are worked in ``splits`` parts
    side by side, whose sums are added in order. Head sizes that fill whole 16-byte words"""
    _need_cuda(q, out, bias, pool, table)
    assert q.shape[0] == B and q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == pool.dtype
    assert pool.is_contiguous() and hd * pool.element_size() % 16 == 0 and splits >= 1
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.shape[0] == nh)
    part = torch.empty((B, nh, splits, hd), dtype=torch.float32, device=q.device) if splits > 1 else None
    _check(load().kb_sigattn_decode(_p(q), dt(q), q.stride(0), _p(out), out.stride(0), _p(part), _p(slot), _p(kv_len),
                                    B, nh, nkv, hd, float(scale), _p(bias), bias.shape[1] if bias is not None else 0,
                                    _p(pool), _p(table), table.stride(0), n_pages, splits, _p(status), _stream()),
           "sigattn_decode")
    if splits > 1:
        add_launches(1)


def sigattn_tc(q: torch.Tensor, out: torch.Tensor, slot, q_start, kv_len, B: int, nh: int, nkv: int, hd: int,
               scale: float, bias: Optional[torch.Tensor], pool: torch.Tensor, table: torch.Tensor, n_pages: int, *,
               grid_x: int, status: torch.Tensor) -> None:
    """attention without a softmax for prompt-sized steps on the tcgen05 kernel (bf16, head size 64 or 128; weights are
    rounded to bf16 for the product with the values): grid_x = ceil(most rows of a sequence / (128 // (nh / nkv)))"""
    _need_cuda(q, out, bias, pool, table)
    assert q.dtype == out.dtype == pool.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert pool.is_contiguous() and hd in (64, 128)
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.shape[0] == nh)
    _check(load().kb_sigattn_tc(_p(q), q.stride(0), _p(out), out.stride(0), _p(slot), _p(q_start), _p(kv_len), B, nh,
                                nkv, hd, float(scale), _p(bias), bias.shape[1] if bias is not None else 0, _p(pool),
                                _p(table), table.stride(0), n_pages, grid_x, _p(status), _stream()), "sigattn_tc")


# ------------------------------------------------------------------------------- per-head steps, norm on the output
def headnorm_rope_store(qkv: torch.Tensor, qout: torch.Tensor, gq: Optional[torch.Tensor], gk: Optional[torch.Tensor],
                        eps: float, dim_true: int, norm: str, inv_freq: Optional[torch.Tensor],
                        inv_freq64: Optional[torch.Tensor], rot: int, t_coef: float, t_every: int, pos, seq, slot,
                        nh: int, nkv: int, nkv_store: int, hd: int, pool: Optional[torch.Tensor], table: torch.Tensor,
                        n_pages: int, status: torch.Tensor) -> None:
    """every query and key head of a row through its OWN root-mean-square norm over ``dim_true`` elements (``norm``:
    "none", "before" or "after" the rotation; gains ``gq`` / ``gk`` float32 [hd] shared by the heads, None for a unit
    norm), the rotation of the pairs (i, i + rot/2), and on queries the temperature ``1 + t_coef ln(floor((pos + 1) /
    t_every) + 1)``; queries to ``qout``, keys and values into their pages. qkv: rows or 32-bit planes of [q heads |
    k heads | v heads]. float32 rows rotate by ``inv_freq64`` (float64), everything else by ``inv_freq``"""
    _need_cuda(qkv, qout, gq, gk, inv_freq, inv_freq64, pool, table)
    planes = qkv.shape[0] if qkv.dim() == 3 else 1
    T = qkv.shape[-2]
    assert qkv.stride(-1) == 1 and qkv.shape[-1] >= (nh + 2 * nkv) * hd and qout.stride(1) == 1
    for g in (gq, gk):
        assert g is None or (g.dtype == torch.float32 and g.numel() == hd and g.is_contiguous())
    assert (gq is None) == (gk is None)
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() >= rot // 2)
    assert inv_freq64 is None or (inv_freq64.dtype == torch.float64 and inv_freq64.numel() >= rot // 2)
    if nkv_store:
        assert pool is not None and pool.dtype == qout.dtype and pool.is_contiguous() and nkv_store == nkv
    pstride = qkv.stride(0) if qkv.dim() == 3 else 0
    mode = {"none": 0, "before": 1, "after": 2}[norm]
    rc = load().kb_headnorm_rope_store(_p(qkv), dt(qkv), planes, pstride, qkv.stride(-2), _p(qout), dt(qout),
                                       qout.stride(0), _p(gq), _p(gk), float(eps), int(dim_true), mode, _p(inv_freq),
                                       _p(inv_freq64), int(rot), float(t_coef), int(t_every), _p(pos), _p(seq),
                                       _p(slot), T, nh, nkv, nkv_store, hd, _p(pool), _p(table), table.stride(0),
                                       n_pages, _p(status), _stream())
    _check(rc, "headnorm_rope_store")


def diff_combine(a: torch.Tensor, out: torch.Tensor, H: int, r: int, hd: int, vd: int, lam: float, eps: float,
                 mult: float) -> None:
    """out[t][h] = unit-RMS(a[t][g][0][i] - lam a[t][g][1][i]) * mult over the head's first ``vd`` values (zero
    beyond), h = g r + i; ``a`` holds 2 H heads of ``hd`` in the order (group, map, head of the group)"""
    _need_cuda(a, out)
    T = a.shape[0]
    assert a.shape[1] == 2 * H * hd and out.shape == (T, H * hd) and a.stride(1) == 1 and out.stride(1) == 1
    assert a.dtype == out.dtype
    _check(load().kb_diff_combine(_p(a), dt(a), a.stride(0), _p(out), out.stride(0), T, H, r, hd, vd, float(lam),
                                  float(eps), float(mult), _stream()), "diff_combine")


def head_gate_mul(a: torch.Tensor, g: torch.Tensor, out: torch.Tensor, hd: int) -> None:
    """out[t][h hd + c] = a[t][h hd + c] * sigmoid(g[t][h]); ``g``: rows [T, >= H] or 32-bit planes [S, T, >= H]"""
    _need_cuda(a, g, out)
    T, N = a.shape
    n_planes, pstride, ldg = _planes_of(g)
    assert N % hd == 0 and g.shape[-1] >= N // hd and g.shape[-2] == T and out.shape == (T, N)
    assert a.stride(1) == 1 and out.stride(1) == 1 and out.dtype == a.dtype
    _check(load().kb_head_gate_mul(_p(a), dt(a), a.stride(0), _p(g), dt(g), n_planes, pstride, ldg, _p(out),
                                   out.stride(0), T, N, hd, _stream()), "head_gate_mul")


def postnorm_add(x: torch.Tensor, delta: torch.Tensor, bias: Optional[torch.Tensor], w: torch.Tensor,
                 ls: Optional[torch.Tensor], eps: float, y: Optional[torch.Tensor]) -> None:
    """x += ls * (w * rms(sum of the planes ``delta`` [S, T, E] + bias)), in place; ``y`` (when given, [T, E] in a run
    dtype) receives the new x"""
    _need_cuda(x, delta, bias, w, ls, y)
    T, E = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and delta.dtype == torch.float32 and delta.dim() == 3
    assert delta.shape[1:] == (T, E) and delta.stride(2) == 1 and delta.stride(1) == E
    assert w.numel() == E and w.is_contiguous() and (ls is None or (ls.numel() == E and ls.is_contiguous()
                                                                    and ls.dtype == w.dtype))
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == E and bias.is_contiguous())
    assert y is None or (y.shape == (T, E) and y.is_contiguous())
    _check(load().kb_postnorm_add(_p(x), _p(delta), delta.shape[0], delta.stride(0), _p(bias), _p(w), _p(ls), dt(w),
                                  float(eps), _p(y), dt(y) if y is not None else F32, T, E, _stream()), "postnorm_add")


def cast_rows(x: torch.Tensor, y: torch.Tensor) -> None:
    """y = x (float32, contiguous) in y's dtype"""
    _need_cuda(x, y)
    assert x.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and y.shape == x.shape
    _check(load().kb_cast_rows(_p(x), _p(y), dt(y), x.numel(), _stream()), "cast_rows")


def glu_clamp(gu: torch.Tensor, out: torch.Tensor, group: int, limit: float, alpha: float) -> None:
    """out = g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit); ``gu``: rows
    [R, 2F] or 32-bit planes [S, R, 2F], gate and up columns in groups of ``group`` (group = F: all gates, then all
    ups)"""
    _need_cuda(gu, out)
    R, F = out.shape
    n_planes, pstride, ldg = _planes_of(gu)
    assert gu.shape[-2] == R and gu.shape[-1] == 2 * F and out.stride(1) == 1 and F % group == 0
    _check(load().kb_glu_clamp(_p(gu), dt(gu), n_planes, pstride, ldg, _p(out), dt(out), out.stride(0), R, F, group,
                               float(limit), float(alpha), _stream()), "glu_clamp")


def moe_route(logits: torch.Tensor, correction: Optional[torch.Tensor], n: int, top: int, groups: int, keep: int):
    """the pick of a router that scores by the softmax over all its ``n`` outputs (the first n columns of float32
    ``logits``): choice by score + ``correction`` inside the ``keep`` best of ``groups`` groups of neighbours, weights
    the chosen scores over their sum: (idx int32 [T, top], weights float32 [T, top])"""
    _need_cuda(logits, correction)
    T = logits.shape[0]
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[1] >= n
    if correction is not None:
        assert correction.dtype == torch.float32 and correction.numel() == n and correction.is_contiguous()
    if n > 256 or groups > 32 or n % groups or not (1 <= keep <= groups) or not (1 <= top <= min(32, n)):
        raise KernelError("kindi_b200: the grouped router pick takes up to 256 outputs in up to 32 equal groups and "
                          "up to 32 picks a row; found %d outputs, %d groups (keep %d), top %d" % (n, groups, keep, top))
    idx = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    wts = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    _check(load().kb_moe_route(_p(logits), logits.stride(0), _p(correction), T, n, top, groups, keep, _p(idx),
                               _p(wts), _stream()), "moe_route")
    return idx, wts


def moe_identity(y: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, planes: torch.Tensor, n_experts: int) -> None:
    """planes[k][t] = wts[t][k] * y[t] for every pick that names an index from ``n_experts`` on (an expert that hands
    its input through); picks below are left as they are"""
    _need_cuda(y, idx, wts, planes)
    T, width = y.shape
    top = idx.shape[1]
    assert y.stride(1) == 1 and idx.is_contiguous() and wts.is_contiguous() and idx.shape == wts.shape == (T, top)
    assert planes.dtype == torch.float32 and planes.shape == (top, T, width) and planes.stride(2) == 1
    assert planes.stride(1) == width
    _check(load().kb_moe_identity(_p(y), dt(y), y.stride(0), _p(idx), _p(wts), _p(planes), planes.stride(0), T * top,
                                  top, n_experts, width, _stream()), "moe_identity")
