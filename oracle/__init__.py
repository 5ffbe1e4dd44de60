"""CPU restatement of the reference's kernels -- test infrastructure only (see oracle.c)."""
