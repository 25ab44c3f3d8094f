"""Drop-in for the reference's `configs` module (benchmark.py:9 does `from configs import *`).  The reference's file
builds the Triton autotune list and asks the GPU driver for its backend while it is imported (configs.py:7-8,17);
the sm_100a operators have no autotuner -- the one knob that changes results, BLOCK_N, is their explicit argument G --
so this module only keeps the names importable."""
import pytest      # noqa: F401  (re-exported, as the reference's module does)
import torch       # noqa: F401


def is_hip():
    return False


configs = []


def keep(conf):
    return True
