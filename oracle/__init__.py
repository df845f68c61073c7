"""CPU oracle for the W4A4 path -- test infrastructure only (see w4a4_oracle.c)."""
