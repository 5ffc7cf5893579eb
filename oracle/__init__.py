"""CPU oracle for the weight-only quantised GEMM path (test infrastructure only)."""
