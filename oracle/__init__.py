"""CPU oracle (test infrastructure; never imported by the product path)."""
