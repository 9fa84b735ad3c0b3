"""CPU oracle for the weight-placement path (test infrastructure only)."""
