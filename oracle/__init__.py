"""CPU oracle for the decode path (test infrastructure; never imported by the product package)."""
