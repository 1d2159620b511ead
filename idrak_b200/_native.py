"""ctypes binding of ``libidrak_b200.so`` (the sm_100a kernels and the C++ runtime).

The library exports a flat C ABI. Every launcher takes raw device pointers and a
``cudaStream_t`` and returns 0 or an error code; :func:`check` turns a non-zero
code into an exception, and :func:`check_status` reads the host-mapped status
word the kernels' bounded waits report into.

On a machine with a GPU the library must be present: :func:`lib` raises rather
than letting a caller fall back to another implementation silently.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_LIB = None
_LOCK = threading.Lock()

c_void_p, c_int, c_float, c_ll = C.c_void_p, C.c_int, C.c_float, C.c_longlong

STATUS_NAMES = {
    0: "ok",
    1: "timeout: a shared-memory stage never filled (TMA copy did not land)",
    2: "timeout: a shared-memory stage was never released",
    3: "timeout: an accumulator never completed",
    4: "timeout: an accumulator was never drained",
    5: "timeout: a peer rank's flag never reached the expected epoch",
    6: "timeout: generic wait",
    7: "bad argument detected on the device",
}

_SIGNATURES = {
    "idrak_status_take": (c_int, [C.POINTER(C.c_uint32)]),
    "idrak_sm_count": (c_int, []),
    "idrak_last_error": (C.c_char_p, []),
    "idrak_launch_count": (c_ll, []),
    "idrak_bind_device": (c_int, [c_int]),
    "idrak_build_info": (C.c_char_p, []),
    "idrak_device_limits": (c_int, [C.POINTER(c_ll), c_int]),
    "idrak_gemm_workspace_elems": (c_ll, [c_int, c_int, c_int, c_int]),
    "idrak_gemm_pick_splits": (c_int, [c_int, c_int, c_int, c_int]),
    "idrak_gemm_bf16": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                                c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int,
                                c_int, c_float, c_int, c_void_p, c_int, c_void_p]),
    "idrak_norm_fwd": (c_int, [c_void_p] * 8 + [c_int, c_int, c_float, c_int, c_void_p]),
    "idrak_norm_bwd_blocks": (c_int, [c_int]),
    "idrak_norm_bwd": (c_int, [c_void_p] * 11 + [c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "idrak_norm_bwd_fused": (c_int, [c_void_p] * 11 + [c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "idrak_norm_bwd_sums_dx": (c_int, [c_int, c_int]),
    "idrak_colsum_blocks": (c_int, [c_int]),
    "idrak_colsum": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "idrak_gelu_fwd": (c_int, [c_void_p, c_void_p, c_ll, c_void_p]),
    "idrak_gelu_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_void_p]),
    "idrak_gated_fwd": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "idrak_gated_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "idrak_add": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_void_p]),
    "idrak_f32_to_bf16": (c_int, [c_void_p, c_void_p, c_ll, c_void_p]),
    "idrak_bf16_to_f32": (c_int, [c_void_p, c_void_p, c_ll, c_void_p]),
    "idrak_rope": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int,
                           c_void_p]),
    "idrak_embedding_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "idrak_wpe_bwd": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "idrak_wte_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "idrak_softmax_xent": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int,
                                   c_int, c_void_p]),
    "idrak_sum_rows": (c_int, [c_void_p, c_int, c_float, c_void_p, c_void_p]),
    "idrak_opt_chunk_elems": (c_int, []),
    "idrak_opt_tensor_bytes": (c_int, []),
    "idrak_opt_chunk_bytes": (c_int, []),
    "idrak_opt_hyper_floats": (c_int, []),
    "idrak_opt_grad_norm": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "idrak_opt_adamw": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "idrak_opt_sgd": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_float, c_int, c_void_p]),
    "idrak_flash_fwd": (c_int, [c_void_p] * 5 + [c_int] * 6 + [c_ll] * 7 + [c_float, c_int, c_void_p]),
    "idrak_flash_bwd": (c_int, [c_void_p] * 10 + [c_int] * 6 + [c_ll] * 9 + [c_float, c_int, c_void_p]),
    "idrak_route_capacity": (c_int, [c_int, c_int, c_int]),
    "idrak_route_blocks": (c_int, [c_int]),
    "idrak_route_choose": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "idrak_route_plan": (c_int, [c_void_p, c_int, c_int, c_int] + [c_void_p] * 9),
    "idrak_route_gather": (c_int, [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "idrak_route_combine": (c_int, [c_void_p] * 6 + [c_int, c_int, c_int, c_void_p, c_void_p]),
    "idrak_gemm_grouped_rows": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_void_p, c_void_p, c_void_p]),
    "idrak_gemm_grouped_k": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_void_p, c_void_p]),
    "idrak_skinny_gemm": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                  c_void_p, c_int, c_int, c_float, c_void_p]),
    "idrak_skinny_splits": (c_int, [c_int, c_int]),
    "idrak_skinny8_gemm": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                   c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "idrak_flash_fwd_ex": (c_int, [c_void_p] * 5 + [c_int] * 6 + [c_ll] * 7 + [c_float, c_int, c_int, c_void_p, c_float,
                                                                              c_void_p]),
    "idrak_gemm_lowrank": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                   c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "idrak_pw_unary": (c_int, [c_int, c_int, c_void_p, c_void_p, c_ll, c_float, c_float, c_void_p]),
    "idrak_pw_unary_bwd": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_ll, c_float, c_float, c_int, c_void_p]),
    "idrak_pw_binary": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_ll, c_float, c_float, c_void_p]),
    "idrak_pw_muladd": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_void_p]),
    "idrak_pw_extremum_bwd": (c_int, [c_int] + [c_void_p] * 5 + [c_ll, c_int, c_void_p]),
    "idrak_pw_where": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_void_p]),
    "idrak_pw_fill": (c_int, [c_int, c_void_p, c_ll, c_float, c_void_p]),
    "idrak_pw_add_rowvec": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p]),
    "idrak_pw_dropout": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_ll, c_float, C.c_ulonglong, c_void_p]),
    "idrak_softmax": (c_int, [c_int, c_void_p, c_void_p, c_ll, c_int, c_float, c_void_p, c_int, c_int, c_int, c_int,
                              c_int, c_void_p]),
    "idrak_softmax_bwd": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_float, c_int, c_void_p]),
    "idrak_sum_axis": (c_int, [c_int, c_void_p, c_void_p, c_ll, c_int, c_ll, c_float, c_void_p]),
    "idrak_broadcast_axis": (c_int, [c_int, c_void_p, c_void_p, c_ll, c_int, c_ll, c_int, c_void_p]),
    "idrak_permute": (c_int, [c_int, c_void_p, c_void_p, c_int, C.POINTER(c_ll), C.POINTER(c_ll), c_void_p]),
    "idrak_transpose": (c_int, [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "idrak_gather_rows": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_ll, c_void_p]),
    "idrak_one_hot": (c_int, [c_int, c_void_p, c_void_p, c_ll, c_int, c_void_p]),
    "idrak_class_match": (c_int, [c_int, c_void_p, c_void_p, c_ll, c_int, c_void_p, c_void_p]),
    "idrak_ctc_alpha_elems": (c_ll, [c_int, c_int, c_int]),
    "idrak_ctc_row_elems": (c_ll, [c_int, c_int]),
    "idrak_ctc_loss": (c_int, [c_void_p] * 7 + [c_int] * 5 + [c_void_p]),
    "idrak_ctc_loss_bwd": (c_int, [c_void_p] * 10 + [c_int] * 5 + [c_void_p]),
    "idrak_lstm_cell": (c_int, [c_int] + [c_void_p] * 5 + [c_int, c_int, c_void_p]),
    "idrak_lstm_cell_bwd": (c_int, [c_int] + [c_void_p] * 7 + [c_int, c_int, c_void_p]),
    "idrak_gru_cell": (c_int, [c_int] + [c_void_p] * 5 + [c_int, c_int, c_void_p]),
    "idrak_gru_cell_bwd": (c_int, [c_int] + [c_void_p] * 6 + [c_int, c_int, c_void_p]),
    "idrak_monotonic_align": (c_int, [c_void_p] * 6 + [c_int, c_int, c_int, c_void_p]),
    "idrak_im2col": (c_int, [c_int, c_void_p, c_void_p, C.POINTER(c_int), c_int, c_void_p]),
    "idrak_col2im": (c_int, [c_int, c_void_p, c_void_p, C.POINTER(c_int), c_int, c_int, c_void_p]),
    "idrak_nchw_to_rows": (c_int, [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "idrak_rows_to_nchw": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "idrak_dw_conv": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, C.POINTER(c_int), c_void_p]),
    "idrak_dw_conv_bwd_input": (c_int, [c_int, c_void_p, c_void_p, c_void_p, C.POINTER(c_int), c_void_p]),
    "idrak_dw_conv_bwd_weight": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, C.POINTER(c_int), c_void_p]),
    "idrak_maxpool": (c_int, [c_int, c_void_p, c_void_p, c_void_p, C.POINTER(c_int), c_void_p]),
    "idrak_maxpool_bwd": (c_int, [c_int, c_void_p, c_void_p, c_void_p, C.POINTER(c_int), c_void_p]),
    "idrak_avgpool": (c_int, [c_int, c_void_p, c_void_p, C.POINTER(c_int), c_int, c_void_p]),
    "idrak_avgpool_bwd": (c_int, [c_int, c_void_p, c_void_p, C.POINTER(c_int), c_int, c_void_p]),
    "idrak_flash_bwd_ex": (c_int, [c_void_p] * 10 + [c_int] * 6 + [c_ll] * 9 + [c_float, c_int, c_int, c_void_p,
                                                                               c_float, c_void_p]),
}


def has(symbol: str) -> bool:
    """Whether the built library exports ``symbol`` (a library older than the Python sources may not)."""
    try:
        getattr(lib(), symbol)
        return True
    except (AttributeError, RuntimeError):
        return False


def lib_path() -> Path:
    """The native library: ``lib/libidrak_b200.so`` beside this file, or the file ``IDRAK_B200_LIB`` names (a build with
    other compile-time options, say)."""
    override = os.environ.get("IDRAK_B200_LIB")
    if override:
        return Path(override).resolve()
    return Path(__file__).resolve().parent / "lib" / "libidrak_b200.so"


def available() -> bool:
    return lib_path().exists()


def lib() -> C.CDLL:
    """The loaded native library. Builds it first when ``IDRAK_B200_AUTOBUILD=1`` and it is missing."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = lib_path()
        if not path.exists():
            if os.environ.get("IDRAK_B200_AUTOBUILD", "0") == "1":
                from . import build as _build
                _build.build()
            else:
                raise RuntimeError(
                    f"native library missing: {path}. Run `python -m idrak_b200.build` "
                    "(or __graft_entry__.build()); the CUDA path has no fallback.")
        handle = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
        for name, (res, args) in _SIGNATURES.items():
            try:
                fn = getattr(handle, name)
            except AttributeError:
                continue
            fn.restype = res
            fn.argtypes = args
        _LIB = handle
        return _LIB


_BOUND_NAMES = set()


def exported_names():
    """Names of the library's entry points this process knows: the signature table plus what modules bound."""
    return sorted(set(_SIGNATURES) | _BOUND_NAMES)


def bind(name: str, restype, argtypes):
    """Declare one more exported function (used by modules that own their part of the ABI)."""
    _BOUND_NAMES.add(name)
    fn = getattr(lib(), name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


class NativeError(RuntimeError):
    pass


_DEBUG_SYNC = None


def _debug_sync() -> bool:
    """``IDRAK_CUDA_DEBUG=1``: synchronise after every native launch and name the call whose kernel failed or gave up a
    bounded wait - what an asynchronous error would otherwise pin on some later call."""
    global _DEBUG_SYNC
    if _DEBUG_SYNC is None:
        import os
        _DEBUG_SYNC = os.environ.get("IDRAK_CUDA_DEBUG", "0") not in ("", "0", "false", "off")
    return _DEBUG_SYNC


def check(rc: int, what: str) -> None:
    if rc == 0:
        if _debug_sync():
            import torch
            if torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing():
                try:
                    torch.cuda.synchronize()
                except RuntimeError as e:
                    raise NativeError(f"{what}: {e}") from None
                check_status(what)
        return
    if rc > 0:
        try:
            import torch
            msg = f"CUDA error {rc}"
            del torch
        except Exception:  # pragma: no cover
            msg = f"CUDA error {rc}"
        raise NativeError(f"{what}: {msg}")
    detail = lib().idrak_last_error()
    raise NativeError(f"{what}: argument error {rc} {detail.decode() if detail else ''}")


def take_status() -> tuple[int, int, int, int]:
    out = (C.c_uint32 * 4)()
    lib().idrak_status_take(out)
    return tuple(int(v) for v in out)  # type: ignore[return-value]


def check_status(what: str = "kernel") -> None:
    """Raise if a bounded wait inside a kernel gave up since the last call. Call after a synchronise."""
    code, where, block, extra = take_status()
    if code:
        raise NativeError(
            f"{what}: device status {code} ({STATUS_NAMES.get(code, '?')}), kernel {where >> 16}, "
            f"site {where & 0xFFFF}, block {block}, extra {extra}")
