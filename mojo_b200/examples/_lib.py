"""ctypes access to the example kernels in libb2kernels.so."""
from __future__ import annotations

import ctypes

import torch

from .. import _ext


class Sphere(ctypes.Structure):
    _fields_ = [(n, ctypes.c_float) for n in ("cx", "cy", "cz", "radius", "r", "g", "b", "albedo0", "albedo1", "specular")]


class Light(ctypes.Structure):
    _fields_ = [(n, ctypes.c_float) for n in ("x", "y", "z", "intensity")]


class Scene(ctypes.Structure):
    _fields_ = [("n_spheres", ctypes.c_int), ("n_lights", ctypes.c_int), ("spheres", Sphere * 8), ("lights", Light * 4)]


def lib():
    L = _ext.kernels_lib()
    L.b2_ex_nbody.restype = ctypes.c_double
    L.b2_ex_nbody.argtypes = [ctypes.c_int64, ctypes.c_double, ctypes.POINTER(ctypes.c_double)]
    return L


def ptr(t: torch.Tensor):
    return ctypes.c_void_p(t.data_ptr())


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def time_cuda(fn, iters=20, warm=3) -> float:
    """Mean milliseconds per call, CUDA events on the launching stream after warm-up."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters
