"""CPU oracle (test infrastructure only; see oracle/c_emit.py)."""
