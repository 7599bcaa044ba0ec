"""apxinf_b200 — B200-native (sm_100a) PI0.5 policy forward behind ApxInf's PI0.5 engine API.

Everything that computes lives in libpi05_b200.so (hand-written CUDA, built in
tree by `python -m apxinf_b200.build`); this package is the Python host-side
mirror of the reference's PI0.5 runtime interface over that library's C ABI.
"""
from ._lib import Pi05Error, lib  # noqa: F401
