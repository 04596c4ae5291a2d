"""CPU oracle for the NVFP4 linear path — TEST INFRASTRUCTURE, not a product path.

Only tests/, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import this package. See ``nvfp4_oracle.cpp`` for the parity status ("parity unpinned" for
the NVFP4 arithmetic; shared conventions pinned against the reference's fixtures).
"""
from .oracle import *  # noqa: F401,F403
