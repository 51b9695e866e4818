"""CPU-only analysis tools that read run records (no training or checkpoint access)."""
