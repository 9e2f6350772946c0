"""CPU oracle for the joint-attention path (test infrastructure, not product code).

Only the tests, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs
import this package, and only as the checker or the timed CPU baseline. The
product package never does.
"""
from .oracle import *  # noqa: F401,F403
