"""B200-native decoder for lmz checkpoint archives.

`lmz_b200.gpu` mirrors the reference's `lmz.gpu` module (same function names,
arguments and error behaviour); `lmz_b200.archive` reads the reference's
archive layout and `lmz_b200.decode` drives whole-archive decode on the GPU.
Importing this package touches neither CUDA nor the compiler.
"""
__version__ = "0.1.0"
