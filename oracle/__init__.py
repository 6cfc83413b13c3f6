"""CPU restatement of the reference's dense attention path and BlockMask construction.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this directory; it is
used by tests/, by __graft_entry__.smoke() and by the cpu_baseline / reference legs of
bench.py, always as the checker or the timed CPU baseline, never as a compute path.
"""
