"""Parallel runtime: process-group bootstrap, tensor-parallel and expert-parallel communicators, symmetric
memory over NVLink/NVSwitch."""
from .dist import DistInfo, init_distributed, host_broadcast_object  # noqa: F401
