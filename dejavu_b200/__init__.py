"""dejavu_b200 — B200-native contextual-sparse decode path with the DejaVu model / operator API.

Compute goes through libdejavu_b200.so (hand-written sm_100a kernels behind the C ABI declared in
include/dejavu_b200.h). Importing the package does not load the library; the first operator call does,
and raises if it has not been built (`python -m dejavu_b200.build`).
"""
__version__ = "0.1.0"
