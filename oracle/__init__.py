"""CPU oracle for the attention path: test infrastructure only (see oracle/oracle.c)."""
