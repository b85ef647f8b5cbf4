"""CPU oracle (test infrastructure).  Only tests, the smoke check and the benchmark's
CPU-baseline leg may import this package; the product library never does."""
