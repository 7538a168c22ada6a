"""CPU oracle for the quantized-linear path. TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import
this package; the product (grilly2_b200) never does. See oracle.c for what
each function restates and how it is pinned.
"""
from .oracle import *  # noqa: F401,F403
