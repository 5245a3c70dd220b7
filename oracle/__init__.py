"""CPU oracle for the attention path (test infrastructure; see oracle.h)."""
