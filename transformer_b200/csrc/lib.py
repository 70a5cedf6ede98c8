"""The compiled kernels as Python callables (ctypes over the library's ``extern "C"`` launchers).

Every launcher returns 0 or an error code; :func:`call` turns a code into an exception that names
the launcher.  Pointers are passed as integers (``tensor.data_ptr()``), and the last argument of
every launcher is the CUDA stream, taken from torch's current stream, so kernels run (and are
captured into CUDA graphs) in order with torch's own work.

The library is loaded on first use and the process fails loudly when it cannot be built or loaded:
there is no CPU path and no library fallback behind these functions.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Dict

import torch

from .build import KernelBuildError, ensure_built

_P, _I, _F, _L, _U = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_ulonglong
_CODES = {"p": _P, "i": _I, "f": _F, "l": _L, "u": _U}

# name -> argument codes (the trailing stream is added for all but the ones marked no_stream)
_SIGNATURES: Dict[str, str] = {
    "tb_embed_f32": "pppii", "tb_embed_bf16": "pppii",
    "tb_add_rmsnorm_f32": "pppppippfpiipi", "tb_add_rmsnorm_bf16": "pppppippfpiipi",
    "tb_add_rmsnorm_router_f32": "pppppippfppppiiii", "tb_add_rmsnorm_router_bf16": "pppppippfppppiiii",
    "tb_rope_cache_f32": "ppppippppiiiii", "tb_rope_cache_bf16": "ppppippppiiiii",
    "tb_attention_f32": "ppppppppppiiiiiiiif", "tb_attention_bf16": "ppppppppppiiiiiiiif",
    "tb_gemm_simt_f32": "pppppliiiiiiii".replace(" ", ""), "tb_gemm_simt_bf16": "pppppliiiiiiii",
    "tb_gemm_skinny_bf16": "pppppliiiiiiiiipii",
    "tb_attention_decode_f32": "ppppppppiiiiiiif", "tb_attention_decode_bf16": "ppppppppiiiiiiif",
    "tb_attention_prefill_bf16": "pppppppppiiiiiif",
    "tb_attention_tc_bf16": "pppppppppiiiiiiiif",
    "tb_gemm_tc_bf16": "ppppiiiiiiii", "tb_gather_rows_bf16": "pppii",
    "tb_attention_decode_mma_bf16": "pppppppppiiiiiiiif",
    "tb_attention_decode_rope_bf16": "pppppppppppiiiiiiiiiif",
    "tb_router_f32": "pppppppppiiii", "tb_router_bf16": "pppppppppiiii",
    "tb_router_rows_bf16": "pppppppppiiii",
    "tb_moe_dispatch": "ppppiii",
    "tb_moe_combine_f32": "ppppiii", "tb_moe_combine_bf16": "ppppiii",
    "tb_sample": "plpiififpp",
    "tb_kernel_status_async": "p",
    "tb_random_fill_f32": "plulf", "tb_random_fill_bf16": "plulf",
}
class TapeArg(ctypes.Union):
    _fields_ = [("p", ctypes.c_void_p), ("i", ctypes.c_int), ("f", ctypes.c_float), ("l", ctypes.c_longlong),
                ("u", ctypes.c_ulonglong)]


TAPE_MAX_ARGS = 24


class TapeEntry(ctypes.Structure):
    """One recorded launcher call (csrc/tape.h)."""
    _fields_ = [("fn", ctypes.c_int), ("n_args", ctypes.c_int), ("ptr_mask", ctypes.c_uint), ("reserved", ctypes.c_int),
                ("args", TapeArg * TAPE_MAX_ARGS)]


class TapeMap(ctypes.Structure):
    """Addresses [base, base + size) of the recorded layer move by delta for the layer being run."""
    _fields_ = [("base", ctypes.c_ulonglong), ("size", ctypes.c_ulonglong), ("delta", ctypes.c_longlong)]


_NO_STREAM = {"tb_attention_tile_tokens": "ii", "tb_gemm_tc_status": "", "tb_attention_prefill_tile_tokens": "",
              "tb_attention_tc_tile_tokens": ""}

_lock = threading.Lock()
_lib = None


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = ensure_built()
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:  # pragma: no cover
                raise KernelBuildError(f"cannot load {path}: {e}") from e
            for name, codes in _SIGNATURES.items():
                fn = getattr(lib, name)
                fn.argtypes = [_CODES[c] for c in codes] + [_P]
                fn.restype = _I
            for name, codes in _NO_STREAM.items():
                fn = getattr(lib, name)
                fn.argtypes = [_CODES[c] for c in codes]
                fn.restype = _I
            lib.tb_tape_index.argtypes = [ctypes.c_char_p]
            lib.tb_tape_index.restype = _I
            lib.tb_tape_replay.argtypes = [ctypes.POINTER(TapeEntry), _I, ctypes.POINTER(TapeMap), _I,
                                           ctypes.POINTER(ctypes.c_int), _P]
            lib.tb_tape_replay.restype = _I
            _lib = lib
    return _lib


def library_path() -> str:
    return ensure_built()


def _error_text(code: int) -> str:
    if code == -1:
        return "bad argument"
    if code == -2:
        return "size not supported by this kernel"
    return f"CUDA error {code}"


launch_count = 0     # launchers called so far (a launcher may start more than one kernel)

_scope_stream = None  # inside stream_scope(): the handle of the stream that was current at its start


class stream_scope:
    """``with stream_scope():`` looks torch's current stream up once for all the launches inside (a model's forward
    pass is some hundred launches, and the look-up costs as much as a launch).  Whoever opens it must not
    change the current stream inside; a scope opened inside a graph capture sees the capturing stream."""

    def __enter__(self):
        global _scope_stream
        self._before = _scope_stream
        _scope_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _scope_stream
        _scope_stream = self._before
        return False


def _stream() -> int:
    return _scope_stream if _scope_stream is not None else torch.cuda.current_stream().cuda_stream


_recorder = None      # while a layer's calls are recorded: an object with launch(name, args) and foreign(kind, *tensors)


class recording:
    """``with recording(tape):`` every launcher call that succeeds inside is also reported to ``tape.launch(name,
    args)``, and device work that does not go through a launcher reports itself with :func:`foreign`."""

    def __init__(self, tape):
        self.tape = tape

    def __enter__(self):
        global _recorder
        self._before = _recorder
        _recorder = self.tape
        return self.tape

    def __exit__(self, *exc):
        global _recorder
        _recorder = self._before
        return False


def foreign(kind: str, *tensors) -> None:
    """Tell a recording that device work of another kind is about to run here (a library product, ...)."""
    if _recorder is not None:
        _recorder.foreign(kind, *tensors)


def try_call(name: str, *args) -> bool:
    """Like :func:`call`, but a kernel that refuses the sizes (TB_ERR_UNSUPPORTED) answers False
    instead of raising, so the caller can take the general kernel."""
    global launch_count
    fn = getattr(_lib if _lib is not None else library(), name)
    rc = fn(*args, _stream())
    if rc == -2:
        return False
    if rc != 0:
        raise KernelError(f"{name}: {_error_text(rc)}")
    launch_count += 1
    if _recorder is not None:
        _recorder.launch(name, args)
    return True


def call(name: str, *args) -> None:
    """Launch ``name`` on torch's current stream."""
    global launch_count
    launch_count += 1
    fn = getattr(_lib if _lib is not None else library(), name)
    rc = fn(*args, _stream())
    if rc != 0:
        raise KernelError(f"{name}: {_error_text(rc)}")
    if _recorder is not None:
        _recorder.launch(name, args)


_tape_indices: Dict[str, int] = {}


def tape_entries(calls) -> "ctypes.Array":
    """[(launcher name, argument tuple)] as the array of TapeEntry that :func:`tape_replay` runs."""
    arr = (TapeEntry * len(calls))()
    for e, (name, args) in zip(arr, calls):
        codes = _SIGNATURES[name]
        if len(args) != len(codes) or len(args) > TAPE_MAX_ARGS:
            raise KernelError(f"{name}: {len(args)} arguments recorded, {len(codes)} declared")
        idx = _tape_indices.get(name)
        if idx is None:
            idx = library().tb_tape_index(name.encode())
            if idx < 0:
                raise KernelError(f"{name} is not registered for replay")
            _tape_indices[name] = idx
        e.fn, e.n_args, mask = idx, len(args), 0
        for j, (c, v) in enumerate(zip(codes, args)):
            if c == "p":
                e.args[j].p = v or None
                mask |= 1 << j
            elif c == "i":
                e.args[j].i = int(v)
            elif c == "f":
                e.args[j].f = float(v)
            elif c == "l":
                e.args[j].l = int(v)
            else:
                e.args[j].u = int(v)
        e.ptr_mask = mask
    return arr


def tape_maps(moves) -> "ctypes.Array":
    """[(base, size, delta)] as an array of TapeMap."""
    arr = (TapeMap * max(1, len(moves)))()
    for m, (base, size, delta) in zip(arr, moves):
        m.base, m.size, m.delta = base, size, delta
    return arr


_failed_at = ctypes.c_int(0)


def tape_replay(entries, maps, n_maps: int) -> None:
    """Run recorded calls on torch's current stream with the pointers of ``maps`` moved."""
    global launch_count
    rc = library().tb_tape_replay(entries, len(entries), maps, n_maps, ctypes.byref(_failed_at), _stream())
    if rc != 0:
        raise KernelError(f"replayed call {_failed_at.value} of {len(entries)}: {_error_text(rc)}")
    launch_count += len(entries)


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def suffix(dtype: torch.dtype) -> str:
    if dtype == torch.float32:
        return "f32"
    if dtype == torch.bfloat16:
        return "bf16"
    raise KernelError(f"kernels exist for float32 and bfloat16, not {dtype}")


def random_fill(t: torch.Tensor, base: int, scale: float, first: int = 0) -> None:
    """Fill the contiguous tensor ``t`` (float32 or bfloat16) with elements first .. first + t.numel() - 1 of the
    counter-based stream that starts at ``base`` (see weights/counter_random.py)."""
    if not t.is_contiguous():
        raise KernelError("random_fill needs a contiguous tensor")
    call("tb_random_fill_" + suffix(t.dtype), t.data_ptr(), t.numel(), int(base), int(first), float(scale))


def attention_tile_tokens(nh: int, nkvh: int) -> int:
    return library().tb_attention_tile_tokens(nh, nkvh)


def gemm_tc_status() -> int:
    """0, or the code of a kernel with bounded waits (the tensor-core products, the tensor-core and the
    page-ring attention) that gave up on a wait since the last call; synchronises the device and clears it."""
    return library().tb_gemm_tc_status()


def kernel_status_async(host_int32: torch.Tensor) -> None:
    """Copy the same code into the first element of a pinned int32 host tensor, in stream order and without
    waiting: it lands together with the step's other results."""
    rc = library().tb_kernel_status_async(host_int32.data_ptr(), _stream())
    if rc != 0:
        raise KernelError(f"tb_kernel_status_async: {_error_text(rc)}")


def _gave_up(code: int) -> str:
    """Which kernel family a wait code belongs to (1..5 tensor-core products, 11..17 tensor-core prompt
    attention, 21..22 decode attention with the page ring)."""
    if 1 <= code <= 5:
        return "tensor-core matrix product"
    if 11 <= code <= 17:
        return "tensor-core prompt attention"
    if 21 <= code <= 22:
        return "decode attention"
    return "unknown kernel"


def raise_for_status(code: int, recover=None) -> None:
    """``code`` is the word the kernels with bounded waits share (0: all well).  Anything else means that a wait
    ran out and the kernel returned early: its result is not to be used.  ``recover()`` is called first (it puts
    back what such a kernel leaves behind), then :class:`KernelError` is raised."""
    if not code:
        return
    if recover is not None:
        recover()
    raise KernelError(f"a kernel gave up after its wait limit (code {code}: {_gave_up(int(code))}); the results of "
                      f"the steps since the last check are not valid")


def attention_prefill_tile_tokens() -> int:
    return library().tb_attention_prefill_tile_tokens()


def attention_tc_tile_tokens() -> int:
    return library().tb_attention_tc_tile_tokens()
