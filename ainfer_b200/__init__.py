"""ainfer_b200: B200-native decode token loop behind the AInfer interfaces.

The product is the native code under csrc/ (CUDA kernels + device C ABI in
libainfer_cuda.so, C++ runtime in libainfer_runtime.so). This package only
binds it for tests and benchmarks; nothing here computes on the CPU.
"""
import os

_M = (1 << 64) - 1


def _mix64(z):
    z = (z + 0x9E3779B97F4A7C15) & _M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    return z ^ (z >> 31)


def fnv1a64(name):
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & _M
    return h


def synth_key(seed, name):
    """Stream key of the synthetic generator for (seed, tensor name)."""
    return _mix64((seed & _M) ^ _mix64(fnv1a64(name)))


def lib_dir():
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")
