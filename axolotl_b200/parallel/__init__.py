"""Parallelism: N-D mesh, symmetric memory, fused compute+collective kernels (FSDP / TP / CP / EP)."""
from .mesh import AXES, DeviceMesh, MeshSpec  # noqa: F401
from .runtime import ParallelRuntime, build_parallel, init_distributed  # noqa: F401
