"""CPU oracle (test infrastructure).  Not imported by the product package."""
