"""CPU oracle for the BPE merge loop (test infrastructure, not product code)."""
