"""CPU oracle of the NVFP4 linear op.  Test infrastructure only: imported by
tests/, __graft_entry__.smoke() and the CPU-baseline legs of bench.py."""
