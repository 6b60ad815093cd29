"""CPU checker for the EXL3 path. Test infrastructure only: imported by tests/, by
__graft_entry__.smoke() and by bench.py's CPU-baseline legs, never by the package."""
