"""CPU oracle for the KV-cache hot path: test infrastructure, never imported by product code."""
