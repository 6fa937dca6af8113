"""pace_b200 - B200 (sm_100a) KV-cache hot path behind PACE's cache-manager and attention-op API.

Host side only: every computation is a hand-written CUDA kernel in
libpace_b200.so, reached through the C ABI of include/pace_b200.h.  There is no
CPU path; importing `pace_b200._C` raises if the library has not been built
(python amd-pace_b200/build.py).
"""
__version__ = "0.1.0"
