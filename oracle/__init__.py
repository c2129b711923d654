"""CPU oracle for the PRICHS MoE-layer forward path: test infrastructure only (see oracle/oracle.py)."""
