"""nntile_b200 - B200 (sm_100a) kernels for NNTile's tiled SDPA path.

The product is the CUDA library ``csrc/libnntile_b200.so`` and its C ABI
(``include/nntile_b200.h``).  This package is the thin host-side mirror of the
reference's operator interface for the path, used by the tests and the
benchmark: ``ops`` (kernel level, argument order of
``nntile::kernel::<op>::cuda<T>``), ``sdpa.Sdpa`` (the order of operations of
``nntile.layer.Sdpa``), ``decode`` and ``parallel`` (sharding of independent
attention units over one process per GPU).

PyTorch is used for device memory and streams only.  There is no CPU fallback:
importing ``ops`` fails loudly when the CUDA library has not been built.
"""
__version__ = "0.1.0"
