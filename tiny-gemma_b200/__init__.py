"""tiny-gemma int8 inference hot path, B200-native.

The directory name has a hyphen, so import it with
``importlib.import_module("tiny-gemma_b200")``; submodules: ``capi`` (ctypes
binding of the C-ABI library), ``build`` (nvcc recipe), ``synth`` (seeded
random weights in the ``gemma_i8.bin`` layout).
"""
