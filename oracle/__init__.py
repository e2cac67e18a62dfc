"""CPU checkers for the PQ2_0 hot path (test infrastructure only; see oracle/oracle.py)."""
