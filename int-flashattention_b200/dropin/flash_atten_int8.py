"""Drop-in for the reference module of the same name (benchmark.py:12)."""
from _pkg import pkg as _pkg

attention_int8 = _pkg.attention_int8
