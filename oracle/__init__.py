"""Test infrastructure only: CPU checkers for the compiled training-step path.

Nothing in the `trainkernel_b200` package imports this directory.  It is used
by `tests/`, by `__graft_entry__.smoke()` and by the CPU-baseline legs of
`bench.py`, always as the thing results are compared with or timed beside,
never as the code that produces a result handed to a user.
"""
