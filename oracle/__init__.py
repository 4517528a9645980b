"""CPU checker for the lmz decode path.  Test infrastructure only.

Nothing under ``lmz_b200`` may import this package; it is used by ``tests/``,
by ``__graft_entry__.smoke()`` and by ``bench.py``'s CPU-baseline legs.
"""
