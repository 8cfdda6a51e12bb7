"""CPU oracle for the quantized-KV codec and decode attention.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory: the only permitted callers are the test-suite, the smoke check in
``__graft_entry__`` and the CPU-baseline / reference legs of ``bench.py``.
"""
from .omni_oracle import *  # noqa: F401,F403
