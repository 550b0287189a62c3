"""CPU oracle of the SM120 matmul op: test infrastructure, not product code.
Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs import it."""
