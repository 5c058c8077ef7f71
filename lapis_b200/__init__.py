"""B200-native replacement for the kernels LAPIS's Kokkos emitter produces for CSR
SpMV / SpMM, dense and batched matmul and the PCG solve loop.

``KokkosBackend`` mirrors ``lapis.KokkosBackend`` (python/lapis/KokkosBackend.py in
the LAPIS project); ``device`` is the device-resident layer over torch tensors;
``partition`` / ``dist`` hold the row-block partitioning used on several GPUs.
All compute goes through ``liblapis_b200.so`` (hand-written sm_100a CUDA behind a C
ABI, see include/lapis_b200.h); there is no CPU path.
"""
from . import KokkosBackend  # noqa: F401

__all__ = ["KokkosBackend"]
