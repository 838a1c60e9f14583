"""B200-native decode hot path behind the reference runtime's operator API.

The product is the shared library built from ``csrc/`` (hand-written sm_100a
kernels + the C ABI declared in ``include/fl_b200.h``). The Python modules here
are the host-side harness over that ABI:

  build    compile the library in-tree with nvcc
  capi     ctypes binding of every entry point (fails loudly if the library or
           a CUDA device is missing; there is no CPU path)
  decoder  mirror of the reference's ``Decoder`` interface for the Llama shape
  synth    seeded synthetic tensors with the shapes and value distributions of
           the benchmark configurations
"""
__all__ = ["build", "capi", "decoder", "synth"]
