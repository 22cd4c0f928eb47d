"""CPU oracle for the FP8 W8A8 hot path: test infrastructure, never imported by the product."""
