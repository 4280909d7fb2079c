"""TEST INFRASTRUCTURE: CPU restatements of the reference's algorithms.  Imported
by tests/, by the smoke check and by the benchmark's CPU-baseline leg only."""
