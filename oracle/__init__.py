"""CPU oracle for the B200 path: test infrastructure only (see oracle/oracle.py)."""
