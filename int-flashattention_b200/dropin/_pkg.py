"""Locates the int-flashattention_b200 package for the drop-in modules in this directory."""
import importlib
import os
import sys

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)
pkg = importlib.import_module("int-flashattention_b200")
