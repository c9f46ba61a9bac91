"""CPU oracle and OpenMP baseline (test infrastructure; never imported by mcsparse_b200)."""
