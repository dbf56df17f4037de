"""CPU oracle for the fast_dl hot path: test infrastructure only.

Nothing under fast_dl_b200/ imports this package.  It may be used by tests/, by
__graft_entry__.smoke() and by bench.py's cpu_baseline / reference legs, as the checker
or as the timed CPU baseline -- never as the thing that is measured or shipped.
"""
