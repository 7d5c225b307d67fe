"""Test infrastructure: CPU oracle for the dense-contraction path (see dense_oracle.c)."""
