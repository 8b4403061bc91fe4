"""CPU oracle (test infrastructure).  See naive_attention.py."""
