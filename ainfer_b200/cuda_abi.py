"""ctypes binding of the device C ABI (include/ainfer_cuda.h).

Thin and explicit: device memory, kernels by name, arguments by index, command
lists. Raises AinferError on any non-zero status. There is no fallback: if the
library or a GPU is missing the import of the library / the open of the device
fails loudly.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(_HERE, "lib")
CUDA_LIB = os.path.join(LIB_DIR, "libainfer_cuda.so")

# Every symbol include/ainfer_cuda.h declares, with ctypes signatures.
_vp, _i, _u32, _u64, _sz = C.c_void_p, C.c_int, C.c_uint32, C.c_uint64, C.c_size_t
_pp = C.POINTER(C.c_void_p)


class Control(C.Structure):
    _fields_ = [("token_id", C.c_int32), ("position", C.c_int32),
                ("active_length", C.c_int32), ("selected_token", C.c_int32)]


class DeviceInfo(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("sm_count", C.c_int32), ("cc_major", C.c_int32),
                ("cc_minor", C.c_int32), ("l2_bytes_mb", C.c_int32), ("total_mem", C.c_uint64),
                ("free_mem", C.c_uint64)]


SIGNATURES = {
    "ainfer_device_open": (_i, [_i, _pp]),
    "ainfer_device_close": (_i, [_vp]),
    "ainfer_device_get_info": (_i, [_vp, C.POINTER(DeviceInfo)]),
    "ainfer_last_error": (C.c_char_p, [_vp]),
    "ainfer_mem_alloc": (_i, [_vp, _sz, _sz, _pp]),
    "ainfer_mem_free": (_i, [_vp, _vp]),
    "ainfer_memcpy_h2d": (_i, [_vp, _vp, _vp, _sz]),
    "ainfer_memcpy_d2h": (_i, [_vp, _vp, _vp, _sz]),
    "ainfer_memcpy_d2d": (_i, [_vp, _vp, _vp, _sz]),
    "ainfer_mem_fill": (_i, [_vp, _vp, _i, _sz]),
    "ainfer_host_alloc": (_i, [_vp, _sz, _pp]),
    "ainfer_host_free": (_i, [_vp, _vp]),
    "ainfer_memcpy_h2d_async": (_i, [_vp, _vp, _vp, _sz]),
    "ainfer_memcpy_d2h_async": (_i, [_vp, _vp, _vp, _sz]),
    "ainfer_kernel_get": (_i, [_vp, C.c_char_p, _pp]),
    "ainfer_kernel_release": (_i, [_vp]),
    "ainfer_kernel_count": (_i, []),
    "ainfer_kernel_name": (C.c_char_p, [_i]),
    "ainfer_kernel_query": (_i, [_vp, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "ainfer_kernel_arg_size": (_i, [_vp, _u32, C.POINTER(_sz)]),
    "ainfer_kernel_set_arg": (_i, [_vp, _u32, _sz, _vp]),
    "ainfer_kernel_max_groups": (_i, [_vp, C.POINTER(_u32)]),
    "ainfer_list_create": (_i, [_vp, _pp]),
    "ainfer_list_append_launch": (_i, [_vp, _vp, _u32]),
    "ainfer_list_append_memcpy": (_i, [_vp, _vp, _vp, _sz]),
    "ainfer_list_append_fill": (_i, [_vp, _vp, _i, _sz]),
    "ainfer_list_close": (_i, [_vp]),
    "ainfer_list_launch_count": (_i, [_vp, C.POINTER(_u32)]),
    "ainfer_list_destroy": (_i, [_vp]),
    "ainfer_list_execute": (_i, [_vp]),
    "ainfer_kernel_launch": (_i, [_vp, _vp, _u32]),
    "ainfer_sync": (_i, [_vp, _u64]),
    "ainfer_control_write": (_i, [_vp, _vp, C.POINTER(Control)]),
    "ainfer_control_write_async": (_i, [_vp, _vp, C.POINTER(Control)]),
    "ainfer_event_create": (_i, [_vp, _pp]),
    "ainfer_event_record": (_i, [_vp]),
    "ainfer_event_elapsed_ms": (_i, [_vp, _vp, C.POINTER(C.c_float)]),
    "ainfer_event_destroy": (_i, [_vp]),
    "ainfer_launch_counter": (_i, [_vp, C.POINTER(_u64)]),
    "ainfer_flush_l2": (_i, [_vp]),
    "ainfer_device_stream": (_i, [_vp, _pp]),
    "ainfer_router_topk_static": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_int32, C.c_int32, C.c_int32]),
}

_lib = None


class AinferError(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"ainfer status {status}: {msg}")
        self.status = status


def load():
    """Loads libainfer_cuda.so; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(CUDA_LIB):
            raise ImportError(f"{CUDA_LIB} is missing: build it with `python -m ainfer_b200._build` "
                              "(there is no fallback path)")
        L = C.CDLL(CUDA_LIB, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def device_count(limit=16):
    """Number of GPUs the library can open (ordinals 0..n-1)."""
    n = 0
    while n < limit:
        h = C.c_void_p()
        if load().ainfer_device_open(n, C.byref(h)):
            break
        load().ainfer_device_close(h)
        n += 1
    return n


class Device:
    def __init__(self, ordinal=0):
        self.L = load()
        h = C.c_void_p()
        st = self.L.ainfer_device_open(ordinal, C.byref(h))
        if st:
            raise AinferError(st, (self.L.ainfer_last_error(None) or b"").decode())
        self.h = h
        self._allocs = []

    def check(self, st):
        if st:
            raise AinferError(st, (self.L.ainfer_last_error(self.h) or b"").decode())

    def info(self):
        inf = DeviceInfo()
        self.check(self.L.ainfer_device_get_info(self.h, C.byref(inf)))
        return inf

    def alloc(self, nbytes, align=256):
        p = C.c_void_p()
        self.check(self.L.ainfer_mem_alloc(self.h, nbytes, align, C.byref(p)))
        self._allocs.append(p.value)
        return p.value

    def free(self, ptr):
        self.check(self.L.ainfer_mem_free(self.h, ptr))
        if ptr in self._allocs:
            self._allocs.remove(ptr)

    def upload(self, arr):
        """numpy array -> fresh device buffer; returns the device address."""
        arr = np.ascontiguousarray(arr)
        p = self.alloc(max(arr.nbytes, 16))
        if arr.nbytes:
            self.check(self.L.ainfer_memcpy_h2d(self.h, p, arr.ctypes.data, arr.nbytes))
        return p

    def zeros(self, nbytes):
        p = self.alloc(max(nbytes, 16))
        self.check(self.L.ainfer_mem_fill(self.h, p, 0, max(nbytes, 16)))
        return p

    def copy_d2d(self, dst, src, nbytes):
        self.check(self.L.ainfer_memcpy_d2d(self.h, dst, src, nbytes))

    def write(self, ptr, arr):
        arr = np.ascontiguousarray(arr)
        self.check(self.L.ainfer_memcpy_h2d(self.h, ptr, arr.ctypes.data, arr.nbytes))

    def download(self, ptr, shape, dtype):
        out = np.zeros(shape, dtype)
        if out.nbytes:
            self.check(self.L.ainfer_memcpy_d2h(self.h, out.ctypes.data, ptr, out.nbytes))
        return out

    def fill(self, ptr, byte, nbytes):
        self.check(self.L.ainfer_mem_fill(self.h, ptr, byte, nbytes))

    def kernel(self, name):
        return Kernel(self, name)

    def sync(self, timeout_ns=2**64 - 1):
        self.check(self.L.ainfer_sync(self.h, timeout_ns))

    def launches(self):
        n = C.c_uint64()
        self.check(self.L.ainfer_launch_counter(self.h, C.byref(n)))
        return n.value

    def flush_l2(self):
        self.check(self.L.ainfer_flush_l2(self.h))

    def event(self):
        return Event(self)

    def new_list(self):
        return CommandList(self)

    def close(self):
        if self.h:
            for p in list(self._allocs):
                self.L.ainfer_mem_free(self.h, p)
            self._allocs = []
            self.L.ainfer_device_close(self.h)
            self.h = None


class Kernel:
    """A kernel handle; arguments are set by index in member order."""

    def __init__(self, dev, name):
        self.dev = dev
        self.name = name
        h = C.c_void_p()
        dev.check(dev.L.ainfer_kernel_get(dev.h, name.encode(), C.byref(h)))
        self.h = h
        n, t, it = C.c_int(), C.c_int(), C.c_int()
        dev.check(dev.L.ainfer_kernel_query(h, C.byref(n), C.byref(t), C.byref(it)))
        self.nargs, self.threads, self.items = n.value, t.value, it.value
        self.sizes = []
        for i in range(self.nargs):
            s = C.c_size_t()
            dev.check(dev.L.ainfer_kernel_arg_size(h, i, C.byref(s)))
            self.sizes.append(s.value)

    def set_arg(self, index, value, kind=None):
        """value: int device address / int / float. kind: 'ptr', 'i32', 'u64', 'f32' (guessed from
        the argument size and the Python type when omitted)."""
        size = self.sizes[index] if index < self.nargs else 0
        if kind is None:
            if isinstance(value, float):
                kind = "f32"
            elif size == 8:
                kind = "u64"
            else:
                kind = "i32"
        if kind == "f32":
            v = C.c_float(value)
        elif kind in ("ptr", "u64"):
            v = C.c_uint64(value or 0)
        else:
            v = C.c_int32(value)
        self.dev.check(self.dev.L.ainfer_kernel_set_arg(self.h, index, C.sizeof(v), C.byref(v)))

    def set_args(self, *values):
        for i, v in enumerate(values):
            self.set_arg(i, v)

    def launch(self, groups):
        self.dev.check(self.dev.L.ainfer_kernel_launch(self.dev.h, self.h, groups))

    def __call__(self, groups, *values):
        self.set_args(*values)
        self.launch(groups)


class CommandList:
    def __init__(self, dev):
        self.dev = dev
        h = C.c_void_p()
        dev.check(dev.L.ainfer_list_create(dev.h, C.byref(h)))
        self.h = h

    def append(self, kernel, groups):
        self.dev.check(self.dev.L.ainfer_list_append_launch(self.h, kernel.h, groups))

    def close(self):
        self.dev.check(self.dev.L.ainfer_list_close(self.h))

    def execute(self):
        self.dev.check(self.dev.L.ainfer_list_execute(self.h))

    def destroy(self):
        if self.h:
            self.dev.L.ainfer_list_destroy(self.h)
            self.h = None


class Event:
    def __init__(self, dev):
        self.dev = dev
        h = C.c_void_p()
        dev.check(dev.L.ainfer_event_create(dev.h, C.byref(h)))
        self.h = h

    def record(self):
        self.dev.check(self.dev.L.ainfer_event_record(self.h))

    def elapsed_ms(self, stop):
        ms = C.c_float()
        self.dev.check(self.dev.L.ainfer_event_elapsed_ms(self.h, stop.h, C.byref(ms)))
        return ms.value
