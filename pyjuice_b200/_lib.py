"""ctypes binding of ``libpcx_b200.so`` (the C ABI declared in ``include/pcx_b200.h``).

There is no fallback: if the library is missing or a GPU entry point is called without it, an
exception is raised.  Arguments are raw device pointers (``tensor.data_ptr()``) and plain integers;
the stream is torch's current CUDA stream, so the launches order with torch work and can be captured
into CUDA graphs.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
import threading
from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# PCX_B200_LIB points at another build of the library (e.g. one with development switches compiled in)
LIB_PATH = os.environ.get("PCX_B200_LIB") or os.path.join(_HERE, "csrc", "libpcx_b200.so")

P, I, L, F = c_void_p, c_int, c_int64, c_float

# name -> argument types, in the order of include/pcx_b200.h (the trailing stream is appended below)
SIGNATURES = {
    "pcx_fill_f32": [P, L, F],
    "pcx_scale_f32": [P, L, F],
    "pcx_exp_f32": [P, L],
    "pcx_set_root_flows": [P, P, L, L, I, I],
    "pcx_input_cat_fwd": [P, P, P, I, P, P, P, I, L, L, I],
    "pcx_input_cat_bwd": [P, P, P, I, P, P, P, I, L, L, I, I],
    "pcx_prod_fwd": [P, P, P, P, L, I, I, I],
    "pcx_prod_bwd": [P, P, P, P, L, I, I, I, I],
    "pcx_sum_fwd": [P, P, P, P, P, P, L, I, I, I],
    "pcx_sum_fwd_alg": [P, P, P, P, P, P, L, I, I, I, I, F],
    "pcx_sum_bwd_ele_alg": [P, P, P, P, P, P, P, P, L, I, I, I, I, I, I, F],
    "pcx_sum_bwd_par_alg": [P, P, P, P, P, P, P, P, P, L, I, I, I, I, I, F],
    "pcx_sum_bwd_ele": [P, P, P, P, P, P, P, P, L, I, I, I, I, I],
    "pcx_sum_bwd_par": [P, P, P, P, P, P, P, P, P, L, I, I, I, I],
    "pcx_pack_sum_params": [P, I, L, P],
    "pcx_sum_fwd_packed": [P, P, P, P, P, L, I, I, I],
    "pcx_sum_fwd_fused": [P, P, P, P, P, I, L, I, I, I],
    "pcx_sum_bwd_ele_fused": [P, P, P, P, P, P, P, I, I, L, I, I, I, I, I],
    "pcx_sum_bwd_par_fused": [P, P, P, P, P, P, P, P, P, I, L, I, I, I, I],
    "pcx_sum_fwd_dense": [P, P, P, P, P, P, P, I, P, L, L, I, I, I],
    "pcx_sum_bwd_ele_dense": [P, P, P, P, P, P, P, P, P, I, P, L, L, I, I, I, I, I],
    "pcx_sum_par_dense_stage": [P, P, P, P, P, P, P, P, L, I, I, I, I, I, I],
    "pcx_sum_par_dense_gemm": [P, P, P, P, P, P, P, L, I, I, I],
    "pcx_pack_sm_params": [P, P, P, P, P, L, I, I, I, I, I],
    "pcx_sum_bwd_par_sm": [P, P, P, P, P, P, P, P, P, P, P, L, I, I, I, I, I],
    "pcx_pack_sm_jobs": [P, I, L, P],
    "pcx_sum_fwd_sm": [P, P, P, P, P, P, P, L, I, I, I],
    "pcx_sum_bwd_ele_sm": [P, P, P, P, P, P, P, P, P, I, L, I, I, I, I, I],
    "pcx_sum_chain": [I, P, P, P, I, L, I, I, I, I, I, P, L],
    "pcx_sum_bwd_par_batched": [P, P, P, P, P, I, L, I, I, I, I],
    "pcx_sum_fwd_noalloc": [P, P, P, P, P, P, L, I, I, I],
    "pcx_sum_bwd_ele_packed": [P, P, P, P, P, P, P, L, I, I, I, I, I],
    "pcx_tied_accum": [P, L, L, P, I],
    "pcx_em_sum": [P, P, P, P, P, P, L, I, F, F, I],
    "pcx_em_input_cat": [P, P, P, P, P, P, L, I, F, F, I],
    "pcx_probe_bounded_wait": [I, I],
    "pcx_em_input_cat_t": [P, P, P, P, L, I, F, F],
    "pcx_input_cat_missing": [P, P, P, P, P, P, P, L, F],
    "pcx_input_cat_shadow": [P, P, L, I],
    "pcx_input_cat_fwd_t": [P, P, P, I, P, P, L, I, L, L, I],
    "pcx_input_cat_bwd_t": [P, P, P, P, I, P, P, L, I, L, L, I, I],
    "pcx_input_cat_flush_t": [P, P, P, P, L, I],
    "pcx_sum_fwd_dense2": [P, P, P, P, P, P, I, P, P, I, P, L, L, I, I, I],
    "pcx_sum_bwd_ele_dense2": [P, P, P, P, P, P, P, P, I, I, P, P, I, P, L, L, I, I, I, I, I],
    "pcx_sum_par_dense2_stage": [P, P, P, P, P, P, P, P, I, L, I, I, I, I, I, I],
    "pcx_sum_par_dense2_gemm": [P, P, P, P, P, P, P, L, I, I, I],
}

# entry points without a stream argument
PLAIN = {"pcx_build_arch": [], "pcx_set_sum_mode": [I], "pcx_set_dependent_launch": [I], "pcx_set_stage_event": [P], "pcx_get_status": [], "pcx_clear_status": [],
         "pcx_packed_tile_count": [L, I, I, I, I], "pcx_dense_scratch_bytes": [I, I, I],
         "pcx_sm_packed_bytes": [L, I, I], "pcx_dense2_scratch_bytes": [I, I, I]}
SUM_MODE = 1        # the process default of the arithmetic mode (see set_sum_mode / use_sum_mode)
_tls = threading.local()   # .mode: this thread's override (use_sum_mode); .c_mode: what the library holds for this thread


def sum_mode() -> int:
    """The arithmetic mode of launches made by the calling thread: the override of an enclosing `use_sum_mode`, else
    the process default.  The library keeps the mode per host thread, so two circuits driven from two threads (or
    one circuit inside `use_sum_mode`) never change each other's arithmetic."""
    m = getattr(_tls, "mode", None)
    return SUM_MODE if m is None else m


def _sync_mode(lib) -> None:
    want = sum_mode()
    if getattr(_tls, "c_mode", 1) != want:
        if lib.pcx_set_sum_mode(want) != 0:
            raise PcxError(f"invalid sum mode {want}")
        _tls.c_mode = want


@contextlib.contextmanager
def use_sum_mode(mode: Optional[int]):
    """Run the enclosed calls of this thread in arithmetic mode ``mode`` (None: leave as is)."""
    if mode is None:
        yield
        return
    if mode not in (0, 1, 2):
        raise PcxError(f"invalid sum mode {mode}")
    prev = getattr(_tls, "mode", None)
    _tls.mode = int(mode)
    try:
        yield
    finally:
        _tls.mode = prev

_lib: Optional[ctypes.CDLL] = None

# Launch accounting for benchmarks: COUNT increments on every call; when PROFILE is a list, every launch is
# bracketed by CUDA events on the launching stream and (name, start, end) is appended to it.
COUNT = 0
PROFILE = None
PROFILE_BYTES = {}          # while PROFILE is a list: bytes written by the buffer-clearing entry points, per name


class PcxError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Load the shared library (once) and declare every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise PcxError(f"{LIB_PATH} is missing: build it with `python -m pyjuice_b200.csrc.build` "
                       "(there is no CPU or PyTorch fallback for the circuit kernels)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, args in PLAIN.items():
        fn = getattr(lib, name)
        fn.restype = c_int64 if name in ("pcx_packed_tile_count", "pcx_dense_scratch_bytes", "pcx_sm_packed_bytes",
                                        "pcx_dense2_scratch_bytes") else c_int
        fn.argtypes = list(args)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = c_int
        fn.argtypes = list(args) + [c_void_p]
    _lib = lib
    return lib


def call(name: str, *args) -> None:
    """Invoke one entry point; tensors are passed as device pointers.  The launch goes to the device of the first
    tensor argument, on torch's current stream OF THAT DEVICE (which need not be the current device)."""
    lib = load()
    conv = []
    dev = None
    for a in args:
        if isinstance(a, torch.Tensor):
            if not a.is_cuda:
                raise PcxError(f"{name}: tensor argument is not on a CUDA device (no CPU path exists)")
            if dev is None:
                dev = a.device
            conv.append(a.data_ptr())
        elif a is None:
            conv.append(None)
        else:
            conv.append(a)
    global COUNT
    COUNT += 1
    _sync_mode(lib)
    if dev is not None and dev.index != torch.cuda.current_device():
        with torch.cuda.device(dev):             # the C side reads per-device state (SM count, built-in scratch)
            rc = _invoke(lib, name, conv, args, dev)
    else:
        rc = _invoke(lib, name, conv, args, dev)
    if rc == -2 and name == "pcx_sum_fwd_noalloc":
        raise PcxError(f"{name}: the table needs more pre-split parameter tiles than the library's built-in scratch "
                       "holds (256 tiles of 32 KB); use the packed entry points with a caller-owned buffer instead")
    if rc != 0:
        raise PcxError(f"{name} failed with status {rc}")


def _invoke(lib, name, conv, args, dev) -> int:
    stream = torch.cuda.current_stream(dev).cuda_stream
    if PROFILE is None:
        return getattr(lib, name)(*conv, stream)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if name in ("pcx_fill_f32", "pcx_scale_f32"):
        PROFILE_BYTES[name] = PROFILE_BYTES.get(name, 0) + 4 * int(args[1])
    a.record()
    if name in ("pcx_sum_fwd_dense2", "pcx_sum_bwd_ele_dense2"):
        # two kernels behind one call: the library records `m` between the operand pre-pass and the GEMM
        m = torch.cuda.Event(enable_timing=True)
        m.record()                                       # creates the underlying event (overwritten by the library)
        lib.pcx_set_stage_event(m.cuda_event)
        rc = getattr(lib, name)(*conv, stream)
        lib.pcx_set_stage_event(None)
        b.record()
        PROFILE.append((name + "_prep", a, m))
        PROFILE.append((name, m, b))
        return rc
    rc = getattr(lib, name)(*conv, stream)
    b.record()
    # the dataflow launch serves two operators: tell them apart by its first argument (0 forward, 1 element flows)
    PROFILE.append((name + ("_fwd", "_ele")[args[0]] if name == "pcx_sum_chain" else name, a, b))
    return rc


def set_sum_mode(mode: int) -> None:
    """Process default: 0 = fp32 CUDA cores, 1 = tensor cores with bf16 hi/lo split (default), 2 = tensor cores,
    single bf16.  A circuit's own ``sum_mode`` attribute, or `use_sum_mode`, overrides it per call."""
    global SUM_MODE
    if int(mode) not in (0, 1, 2):
        raise PcxError(f"invalid sum mode {mode}")
    SUM_MODE = int(mode)


def get_status(device=None) -> int:
    """Status word of ``device`` (default: the current device): 0, or the code of the first bounded wait of a
    tensor-core kernel that ran out since the word was last cleared.  Synchronises that device."""
    with torch.cuda.device(device):
        return int(load().pcx_get_status())


def clear_status(device=None) -> None:
    with torch.cuda.device(device):
        rc = load().pcx_clear_status()
    if rc != 0:
        raise PcxError(f"pcx_clear_status failed with status {rc}")


def check_status(device=None) -> None:
    """Raise if a tensor-core kernel on ``device`` reported that one of its bounded barrier waits ran out (its tile
    was skipped, so results computed since are wrong); the word is cleared so that later checks start afresh.

    The library calls this where the host synchronises anyway (`TensorCircuit.update_parameters`, `io.save`, reading
    `_cum_flow`); a training loop that never does any of these should call it itself now and then."""
    code = get_status(device)
    if code != 0:
        clear_status(device)
        raise PcxError(f"a tensor-core kernel gave up waiting on a barrier (status {code})")
