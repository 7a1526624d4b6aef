"""ctypes binding of libh3b200.so.

The prototypes are read from include/h3b200.h, so Python calls the C ABI with exactly
the argument types a C caller of the reference's h3_gpu.h would use. `Gpu` wraps a
context and mirrors the reference's calling pattern: ops return 1/0, the message comes
from h3_gpu_error(), work is bracketed by begin()/submit().

There is no fallback: if the shared library is missing or no sm_100 device is present,
creating a context raises.
"""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
HEADER = HERE.parent / "include" / "h3b200.h"
LIBRARY = HERE / "libh3b200.so"

F32, BF16, I8, U32 = 0, 1, 2, 3
_ITEM = {F32: 4, BF16: 2, I8: 1, U32: 4}
_NP = {F32: np.float32, BF16: np.uint16, I8: np.int8, U32: np.uint32}


class H3Error(RuntimeError):
    pass


class Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in
                ("allocated_bytes", "live_bytes", "peak_live_bytes", "tensor_allocations",
                 "direct_dispatches", "mps_linear_dispatches", "mps_conv_dispatches",
                 "mps_sdpa_dispatches", "blit_copies", "submissions")] + \
               [(n, C.c_double) for n in
                ("command_encode_seconds", "command_wait_seconds", "gpu_seconds")]


class DeviceInfo(C.Structure):
    _fields_ = [("name", C.c_char * 256), ("total_memory", C.c_uint64), ("compute_major", C.c_int),
                ("compute_minor", C.c_int), ("multiprocessors", C.c_int)]


class UlyssesPeers(C.Structure):
    """h3x_ulysses_peers: pointers to every rank's exchange buffers as mapped in this process."""
    _fields_ = [("world", C.c_uint32), ("rank", C.c_uint32), ("rows_local", C.c_uint32)] + \
               [(n, C.c_void_p * 8) for n in ("q", "k", "v", "o", "flags")]


_CTYPES = {
    "void": None, "int": C.c_int, "float": C.c_float, "double": C.c_double,
    "uint32_t": C.c_uint32, "uint64_t": C.c_uint64, "size_t": C.c_size_t,
    "h3_gpu_dtype": C.c_int, "long long": C.c_longlong,
}


def _ctype(text: str):
    text = re.sub(r"\bconst\b", "", text).strip()
    if text.endswith("*"):
        base = text[:-1].strip()
        if base == "char":
            return C.c_char_p
        if base == "h3_gpu_stats":
            return C.POINTER(Stats)
        if base == "h3b200_device_info":
            return C.POINTER(DeviceInfo)
        return C.c_void_p
    return _CTYPES[text]


def declared_functions() -> dict[str, tuple]:
    """name -> (restype, [argtypes]) for every function include/h3b200.h declares."""
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"^[ \t]*#.*$", "", text, flags=re.M)          # preprocessor lines
    text = re.sub(r"typedef\s+(struct|enum)\s*\{.*?\}\s*\w+\s*;", "", text, flags=re.S)
    out = {}
    pattern = re.compile(r"([A-Za-z_][\w\s\*]*?)\b(h3x?_\w+|h3b200_\w+)\s*\(([^;{}]*?)\)\s*;", re.S)
    for ret, name, args in pattern.findall(text):
        ret = ret.strip()
        if ret.startswith("typedef"):
            continue
        argtypes = []
        args = " ".join(args.split())
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                m = re.match(r"(.*?)(\w+)$", a)   # strip the parameter name
                argtypes.append(_ctype(m.group(1) if m and m.group(1).strip() else a))
        out[name] = (_ctype(ret), argtypes)
    return out


_libs: dict[str, C.CDLL] = {}


def library(path: str | Path | None = None) -> C.CDLL:
    """libh3b200.so by default. Any other library that exports the reference's h3_gpu_*
    ABI (e.g. the reference's own CUDA backend built as a checker) can be loaded the same
    way; symbols it lacks are simply left unbound."""
    path = Path(path) if path else LIBRARY
    key = str(path)
    if key not in _libs:
        if not path.exists():
            raise H3Error(f"{path} is missing: run `python h3.c_b200/build.py` "
                          "(there is no CPU fallback)")
        lib = C.CDLL(key)
        for name, (restype, argtypes) in declared_functions().items():
            try:
                fn = getattr(lib, name)
            except AttributeError:
                if path == LIBRARY:
                    raise
                continue
            fn.restype = restype
            fn.argtypes = argtypes
        _libs[key] = lib
    return _libs[key]


class Tensor:
    """A device tensor owned by (or wrapped into) a context."""

    def __init__(self, gpu: "Gpu", handle: int, elements: int, dtype: int):
        if not handle:
            raise H3Error(f"tensor allocation failed: {gpu.error()}")
        self.gpu, self.handle, self.elements, self.dtype = gpu, handle, elements, dtype

    @property
    def pointer(self) -> int:
        return self.gpu.lib.h3x_tensor_device_pointer(self.handle)

    def read(self, elements: int | None = None) -> np.ndarray:
        n = self.elements if elements is None else elements
        out = np.empty(n, _NP[self.dtype])
        lib = self.gpu.lib
        if self.dtype == F32:
            ok = lib.h3_gpu_tensor_read_f32(self.handle, out.ctypes.data, n)
        elif self.dtype == BF16:
            ok = lib.h3_gpu_tensor_read_bf16(self.handle, out.ctypes.data, n)
        else:
            raise H3Error("only F32 and BF16 tensors can be read back through the API")
        if not ok:
            raise H3Error("tensor read failed")
        return out

    def write(self, values: np.ndarray, offset: int = 0) -> None:
        values = np.ascontiguousarray(values, _NP[self.dtype]).reshape(-1)
        lib = self.gpu.lib
        if self.dtype == F32:
            ok = lib.h3_gpu_tensor_write_f32_range(self.handle, offset, values.ctypes.data, values.size)
        elif self.dtype == BF16:
            ok = lib.h3_gpu_tensor_write_bf16_range(self.handle, offset, values.ctypes.data, values.size)
        else:
            raise H3Error("only F32 and BF16 tensors can be written through the API")
        if not ok:
            raise H3Error("tensor write failed")

    def free(self) -> None:
        if self.handle:
            self.gpu.lib.h3_gpu_tensor_free(self.handle)
            self.handle = 0


class Gpu:
    """One context = one device + one in-order stream (reference: h3_gpu)."""

    def __init__(self, device: int = 0, lib_path: str | Path | None = None):
        lib = library(lib_path)
        if hasattr(lib, "h3x_set_device") and not lib.h3x_set_device(device):
            raise H3Error(f"no CUDA device {device} (libh3b200 has no CPU fallback)")
        err = C.create_string_buffer(512)
        self.handle = lib.h3_gpu_create(None, err, len(err))
        if not self.handle:
            raise H3Error(f"h3_gpu_create failed: {err.value.decode()}")
        self.lib = lib
        self.device = device

    # ---- lifecycle
    def close(self):
        if self.handle:
            self.lib.h3_gpu_free(self.handle)
            self.handle = 0

    def error(self) -> str:
        return self.lib.h3_gpu_error(self.handle).decode()

    def begin(self):
        if not self.lib.h3_gpu_begin(self.handle):
            raise H3Error("h3_gpu_begin failed (command already active?)")

    def submit(self):
        if not self.lib.h3_gpu_submit(self.handle):
            raise H3Error(f"h3_gpu_submit failed: {self.error()}")

    def flush(self):
        self.lib.h3_gpu_continue(self.handle)

    def stats(self) -> Stats:
        s = Stats()
        self.lib.h3_gpu_get_stats(self.handle, C.byref(s))
        return s

    def set_stream(self, cuda_stream: int):
        if not self.lib.h3x_set_stream(self.handle, cuda_stream):
            raise H3Error(self.error())

    # ---- tensors
    def new(self, elements: int, dtype: int) -> Tensor:
        fn = {F32: self.lib.h3_gpu_tensor_new_f32, BF16: self.lib.h3_gpu_tensor_new_bf16,
              I8: self.lib.h3_gpu_tensor_new_i8}[dtype]
        return Tensor(self, fn(self.handle, elements), elements, dtype)

    def upload(self, values: np.ndarray, dtype: int) -> Tensor:
        values = np.ascontiguousarray(values, _NP[dtype]).reshape(-1)
        fn = {F32: self.lib.h3_gpu_tensor_from_f32, BF16: self.lib.h3_gpu_tensor_from_bf16,
              U32: self.lib.h3_gpu_tensor_from_u32}[dtype]
        return Tensor(self, fn(self.handle, values.ctypes.data, values.size), values.size, dtype)

    def bf16(self, values) -> Tensor:
        return self.upload(values, BF16)

    def f32(self, values) -> Tensor:
        return self.upload(values, F32)

    def u32(self, values) -> Tensor:
        return self.upload(values, U32)

    def wrap(self, device_pointer: int, elements: int, dtype: int) -> Tensor:
        return Tensor(self, self.lib.h3x_tensor_wrap(self.handle, device_pointer, elements, dtype),
                      elements, dtype)

    # ---- ops: gpu.op("linear_bf16", out, x, w, None, rows, k, n) calls h3_gpu_linear_bf16
    def op(self, name: str, *args) -> None:
        fn = getattr(self.lib, name if name.startswith("h3") else "h3_gpu_" + name)
        raw = [a.handle if isinstance(a, Tensor) else C.byref(a) if isinstance(a, C.Structure)
               else a for a in args]
        if not fn(self.handle, *raw):
            raise H3Error(f"{name} failed: {self.error()}")

    def try_op(self, name: str, *args) -> bool:
        fn = getattr(self.lib, name if name.startswith("h3") else "h3_gpu_" + name)
        raw = [a.handle if isinstance(a, Tensor) else a for a in args]
        return bool(fn(self.handle, *raw))
