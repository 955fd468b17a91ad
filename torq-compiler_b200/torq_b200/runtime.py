"""Python binding of the C ABI in include/torq_b200.h, and an inference runner with
the surface of the reference's `torq.runtime.VMFBInferenceRunner`
(runtime/bindings/python/torq/runtime/vmfb.py:140-285): construct from a model
file, `infer(inputs)`, `infer_time_ms`, optional on-device outputs.

The library is required: importing succeeds without it, but creating a Device
raises. Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import os
import time
from typing import Iterable, Sequence

import numpy as np

from .oplist import DTYPE_SIZE, DTYPES, NP_DTYPE

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtorq_b200.so")

OK = 0
STATUS_NAMES = ["OK", "CANCELLED", "UNKNOWN", "INVALID_ARGUMENT", "DEADLINE_EXCEEDED", "NOT_FOUND", "ALREADY_EXISTS",
                "PERMISSION_DENIED", "RESOURCE_EXHAUSTED", "FAILED_PRECONDITION", "ABORTED", "OUT_OF_RANGE",
                "UNIMPLEMENTED", "INTERNAL", "UNAVAILABLE", "DATA_LOSS"]
MEMORY_DEVICE_LOCAL, MEMORY_HOST_PINNED = 0, 1
_DTYPE_NAME = {v: k for k, v in DTYPES.items()}


class TorqB200Error(RuntimeError):
    def __init__(self, status: int, message: str = ""):
        self.status = status
        self.status_name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"{self.status_name}: {message}" if message else self.status_name)


class Binding(C.Structure):
    _fields_ = [("buffer", C.c_void_p), ("offset", C.c_uint64), ("length", C.c_uint64)]


class IoInfo(C.Structure):
    _fields_ = [("dtype", C.c_uint32), ("rank", C.c_uint32), ("shape", C.c_int32 * 4), ("bytes", C.c_uint64)]


_lib = None

# every symbol include/torq_b200.h declares: (restype, argtypes)
_SIGNATURES = {
    "tb200_device_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "tb200_device_destroy": (C.c_int, [C.c_void_p]),
    "tb200_device_query_i64": (C.c_int, [C.c_void_p, C.c_char_p, C.c_char_p, C.POINTER(C.c_int64)]),
    "tb200_device_stream": (C.c_void_p, [C.c_void_p]),
    "tb200_last_error": (C.c_char_p, [C.c_void_p]),
    "tb200_status_string": (C.c_char_p, [C.c_int]),
    "tb200_device_set_profile_csv": (C.c_int, [C.c_void_p, C.c_char_p]),
    "tb200_buffer_alloc": (C.c_int, [C.c_void_p, C.c_uint64, C.c_int, C.POINTER(C.c_void_p)]),
    "tb200_buffer_import": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.POINTER(C.c_void_p)]),
    "tb200_buffer_free": (C.c_int, [C.c_void_p]),
    "tb200_buffer_upload": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64]),
    "tb200_buffer_download": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64]),
    "tb200_buffer_pointer": (C.c_void_p, [C.c_void_p]),
    "tb200_buffer_size": (C.c_uint64, [C.c_void_p]),
    "tb200_executable_create": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "tb200_executable_destroy": (C.c_int, [C.c_void_p]),
    "tb200_executable_io_count": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "tb200_executable_io_info": (C.c_int, [C.c_void_p, C.c_int, C.c_uint32, C.POINTER(IoInfo)]),
    "tb200_executable_op_count": (C.c_uint32, [C.c_void_p]),
    "tb200_executable_launch_count": (C.c_uint32, [C.c_void_p]),
    "tb200_executable_op_kernel": (C.c_char_p, [C.c_void_p, C.c_uint32]),
    "tb200_dispatch": (C.c_int, [C.c_void_p, C.POINTER(Binding), C.c_size_t]),
    "tb200_wait": (C.c_int, [C.c_void_p, C.c_uint64]),
    "tb200_invoke_host": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "tb200_invoke_host_async": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "tb200_executable_comm_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "tb200_executable_comm_handle": (C.c_int, [C.c_void_p, C.c_void_p]),
    "tb200_executable_connect_peers": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "tb200_gemv_w8_noalloc": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                        C.c_int, C.c_int, C.c_int, C.c_int]),
    "tb200_device_probe_bounded_wait": (C.c_int, [C.c_void_p, C.c_uint32]),
    "tb200_measure_i8_mma_peak": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "tb200_debug_read_gemm_trace": (C.c_int, [C.POINTER(C.c_ulonglong), C.c_int]),
    "tb200_executable_profile_ops": (C.c_int, [C.c_void_p, C.POINTER(Binding), C.c_size_t, C.c_int, C.c_int,
                                               C.POINTER(C.c_float), C.c_uint32]),
}


def load_library() -> C.CDLL:
    """dlopen libtorq_b200.so and bind every declared entry point; raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python torq-compiler_b200/build.py` "
                               "(there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library does not export it
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def exported_symbols() -> list[str]:
    return list(_SIGNATURES)


class Device:
    """One B200 + one stream (iree_hal_torq_device_create, runtime/driver/torq_device.c:80-132)."""

    def __init__(self, ordinal: int = 0):
        self._lib = load_library()
        h = C.c_void_p()
        st = self._lib.tb200_device_create(ordinal, C.byref(h))
        if st != OK:
            raise TorqB200Error(st, f"cannot create device cuda:{ordinal} (an sm_100 GPU is required)")
        self._h = h
        self.ordinal = ordinal

    def _check(self, st: int):
        if st != OK:
            raise TorqB200Error(st, (self._lib.tb200_last_error(self._h) or b"").decode())

    @property
    def stream(self) -> int:
        """cudaStream_t handle of the device's stream (for event timing / interop)."""
        return self._lib.tb200_device_stream(self._h) or 0

    def query_i64(self, category: str, key: str) -> int:
        v = C.c_int64()
        self._check(self._lib.tb200_device_query_i64(self._h, category.encode(), key.encode(), C.byref(v)))
        return v.value

    def set_profile_csv(self, path: str | None):
        self._check(self._lib.tb200_device_set_profile_csv(self._h, path.encode() if path else None))

    def alloc(self, nbytes: int, memory_type: int = MEMORY_DEVICE_LOCAL) -> "Buffer":
        h = C.c_void_p()
        self._check(self._lib.tb200_buffer_alloc(self._h, nbytes, memory_type, C.byref(h)))
        return Buffer(self, h, nbytes, memory_type)

    def import_pointer(self, device_pointer: int, nbytes: int) -> "Buffer":
        h = C.c_void_p()
        self._check(self._lib.tb200_buffer_import(self._h, C.c_void_p(device_pointer), nbytes, C.byref(h)))
        return Buffer(self, h, nbytes, MEMORY_DEVICE_LOCAL)

    def wait(self, timeout_s: float = 60.0):
        self._check(self._lib.tb200_wait(self._h, int(timeout_s * 1e9)))

    def probe_bounded_wait(self, limit_ms: int = 20):
        """Queues a kernel whose (bounded) wait nothing completes: the next wait() raises ABORTED once."""
        self._check(self._lib.tb200_device_probe_bounded_wait(self._h, limit_ms))

    def close(self):
        if self._h:
            self._lib.tb200_device_destroy(self._h)
            self._h = None


class Buffer:
    def __init__(self, device: Device, handle, nbytes: int, memory_type: int):
        self.device, self._h, self.nbytes, self.memory_type = device, handle, nbytes, memory_type

    @property
    def pointer(self) -> int:
        return self.device._lib.tb200_buffer_pointer(self._h) or 0

    def upload(self, array: np.ndarray, offset: int = 0):
        a = np.ascontiguousarray(array)
        self.device._check(self.device._lib.tb200_buffer_upload(self._h, offset, a.ctypes.data_as(C.c_void_p), a.nbytes))
        self._keep = a  # the copy is stream-ordered: keep the source alive until the next wait

    def download(self, shape, dtype, offset: int = 0) -> np.ndarray:
        out = np.empty(shape, dtype)
        self.device._check(self.device._lib.tb200_buffer_download(self._h, offset, out.ctypes.data_as(C.c_void_p), out.nbytes))
        self.device.wait()
        return out

    def as_numpy(self, shape, dtype) -> np.ndarray:
        """View of a HOST_PINNED buffer."""
        if self.memory_type != MEMORY_HOST_PINNED:
            raise ValueError("only pinned host buffers are host visible")
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        raw = (C.c_uint8 * n).from_address(self.pointer)
        return np.frombuffer(raw, dtype=dtype).reshape(shape)

    def free(self):
        if self._h:
            self.device._lib.tb200_buffer_free(self._h)
            self._h = None


class TensorInfo:
    """Shape/dtype of a model input or output (runtime/bindings/python/torq/runtime/utils.py TensorInfo)."""

    def __init__(self, info: IoInfo):
        self.dtype = _DTYPE_NAME[info.dtype]
        self.shape = tuple(info.shape[i] for i in range(info.rank))
        self.nbytes = int(info.bytes)
        self.np_dtype = NP_DTYPE[self.dtype]

    def __repr__(self):
        return f"TensorInfo({'x'.join(map(str, self.shape))}x{self.dtype})"


class Executable:
    """A loaded torq-b200-ops dispatch (native_executable.cc:41-108 + TorqExecutable::initialize)."""

    def __init__(self, device: Device, blob: bytes):
        self.device = device
        h = C.c_void_p()
        buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        device._check(device._lib.tb200_executable_create(device._h, buf, len(blob), C.byref(h)))
        self._h = h
        ni, no = C.c_uint32(), C.c_uint32()
        device._check(device._lib.tb200_executable_io_count(h, C.byref(ni), C.byref(no)))
        self.inputs_info = [self._info(0, i) for i in range(ni.value)]
        self.outputs_info = [self._info(1, i) for i in range(no.value)]

    def _info(self, is_out: int, i: int) -> TensorInfo:
        info = IoInfo()
        self.device._check(self.device._lib.tb200_executable_io_info(self._h, is_out, i, C.byref(info)))
        return TensorInfo(info)

    @property
    def op_count(self) -> int:
        return self.device._lib.tb200_executable_op_count(self._h)

    @property
    def launch_count(self) -> int:
        return self.device._lib.tb200_executable_launch_count(self._h)

    @property
    def comm_info(self) -> tuple[int, int]:
        """(rank, group size) of a tensor-parallel shard; (0, 1) for an ordinary executable."""
        r, n = C.c_int32(), C.c_int32()
        self.device._check(self.device._lib.tb200_executable_comm_info(self._h, C.byref(r), C.byref(n)))
        return r.value, n.value

    def comm_handle(self) -> bytes:
        """This shard's 96-byte handle, to be sent to the other members of the group."""
        buf = C.create_string_buffer(96)
        self.device._check(self.device._lib.tb200_executable_comm_handle(self._h, buf))
        return buf.raw

    def connect_peers(self, handles: Sequence[bytes]):
        """handles: every member's comm_handle(), in rank order (this member's own included)."""
        blob = b"".join(handles)
        if len(blob) != 96 * len(handles):
            raise ValueError("comm handles are 96 bytes each")
        self.device._check(self.device._lib.tb200_executable_connect_peers(self._h, blob, len(handles)))

    def connect_group(self, group=None):
        """Exchanges the handles over torch.distributed (any backend) and connects; every member of
        the group calls it. Ends with a barrier: after it every member may dispatch."""
        import torch.distributed as dist
        rank, size = self.comm_info
        if dist.get_world_size(group) != size or dist.get_rank(group) != rank:
            raise ValueError("the process group does not match the shard's rank and group size")
        handles = [None] * size
        dist.all_gather_object(handles, self.comm_handle(), group=group)
        self.connect_peers(handles)
        dist.barrier(group=group)

    def op_kernels(self) -> list[str]:
        return [self.device._lib.tb200_executable_op_kernel(self._h, i).decode() for i in range(self.op_count)]

    def _bindings(self, buffers: Sequence[Buffer]):
        arr = (Binding * len(buffers))()
        for i, b in enumerate(buffers):
            arr[i].buffer, arr[i].offset, arr[i].length = b._h, 0, 0
        return arr

    def dispatch(self, inputs: Sequence[Buffer], outputs: Sequence[Buffer]):
        """Asynchronous: queues the launches on the device stream."""
        bufs = list(inputs) + list(outputs)
        self.device._check(self.device._lib.tb200_dispatch(self._h, self._bindings(bufs), len(bufs)))

    def invoke_host(self, host_inputs: Sequence[np.ndarray], host_outputs: Sequence[np.ndarray]):
        """Synchronous host-pointer call: H2D, dispatch, D2H, wait."""
        ins = (C.c_void_p * len(host_inputs))(*[a.ctypes.data for a in host_inputs])
        outs = (C.c_void_p * len(host_outputs))(*[a.ctypes.data for a in host_outputs])
        self.device._check(self.device._lib.tb200_invoke_host(self._h, ins, outs))

    def invoke_host_async(self, host_inputs: Sequence[np.ndarray], host_outputs: Sequence[np.ndarray]):
        """As invoke_host without the final wait: the upload overlaps the previous call's kernels.
        Arrays must stay alive (and outputs are defined) only after Device.wait()."""
        ins = (C.c_void_p * len(host_inputs))(*[a.ctypes.data for a in host_inputs])
        outs = (C.c_void_p * len(host_outputs))(*[a.ctypes.data for a in host_outputs])
        self.device._check(self.device._lib.tb200_invoke_host_async(self._h, ins, outs))

    def profile_ops(self, inputs: Sequence[Buffer], outputs: Sequence[Buffer], warmup=1, iters=3) -> np.ndarray:
        bufs = list(inputs) + list(outputs)
        ms = (C.c_float * self.op_count)()
        self.device._check(self.device._lib.tb200_executable_profile_ops(
            self._h, self._bindings(bufs), len(bufs), warmup, iters, ms, self.op_count))
        return np.array(ms[:], np.float32)

    def destroy(self):
        if self._h:
            self.device._lib.tb200_executable_destroy(self._h)
            self._h = None


class InferenceRunner:
    """Loads a `.b200ops` model file (or bytes) and runs it; surface of the reference's
    VMFBInferenceRunner (vmfb.py:140-285): `infer`, `infer_time_ms`, `inputs_info`,
    `outputs_info`, `device_outputs`."""

    def __init__(self, model, *, function: str = "main", device_uri: str = "torq_b200", device: Device | None = None,
                 device_outputs: bool = False, runtime_flags: Iterable[str] | None = None):
        if isinstance(model, (bytes, bytearray)):
            blob = bytes(model)
        else:
            with open(model, "rb") as f:
                blob = f.read()
        if not device_uri.startswith("torq_b200"):
            raise ValueError(f"device_uri {device_uri!r}: this runner drives only torq_b200[:ordinal]")
        ordinal = int(device_uri.split(":")[1]) if ":" in device_uri else 0
        self._own_device = device is None
        self.device = device or Device(ordinal)
        for flag in runtime_flags or ():
            if flag.startswith("--torq_profile_host="):
                self.device.set_profile_csv(flag.split("=", 1)[1])
        self.function = function
        self.executable = Executable(self.device, blob)
        self.inputs_info = self.executable.inputs_info
        self.outputs_info = self.executable.outputs_info
        self._device_outputs = device_outputs
        self._in = [self.device.alloc(i.nbytes) for i in self.inputs_info]
        self._out = [self.device.alloc(o.nbytes) for o in self.outputs_info]
        self.infer_time_ms = None

    def infer(self, inputs: Sequence[np.ndarray]):
        if len(inputs) != len(self.inputs_info):
            raise ValueError(f"model takes {len(self.inputs_info)} inputs, got {len(inputs)}")
        t0 = time.perf_counter()
        for a, info, buf in zip(inputs, self.inputs_info, self._in):
            a = np.ascontiguousarray(a, dtype=info.np_dtype)
            if a.shape != info.shape:
                raise ValueError(f"input shape {a.shape} != {info.shape}")
            buf.upload(a)
        self.executable.dispatch(self._in, self._out)
        if self._device_outputs:
            self.device.wait()
            self.infer_time_ms = (time.perf_counter() - t0) * 1e3
            return list(self._out)
        outs = [b.download(o.shape, o.np_dtype) for b, o in zip(self._out, self.outputs_info)]
        self.infer_time_ms = (time.perf_counter() - t0) * 1e3
        return outs

    def close(self):
        for b in self._in + self._out:
            b.free()
        self.executable.destroy()
        if self._own_device:
            self.device.close()


def measure_i8_mma_peak(ordinal: int = 0, rounds: int = 2000) -> tuple[float, float]:
    """(tera-ops/s, ms) of the resident-operand tcgen05 kind::i8 loop on every SM of GPU `ordinal`."""
    lib = load_library()
    tops, ms = C.c_double(), C.c_double()
    st = lib.tb200_measure_i8_mma_peak(ordinal, rounds, C.byref(tops), C.byref(ms))
    if st != OK:
        raise TorqB200Error(st, "int8 tensor-pipe peak measurement failed")
    return tops.value, ms.value


def run_model(model, inputs: Sequence[np.ndarray], **kw):
    """One-shot helper (`torq.runtime.run_vmfb`, vmfb.py:26-76)."""
    r = InferenceRunner(model, **kw)
    try:
        return r.infer(inputs)
    finally:
        r.close()
