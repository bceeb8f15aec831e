"""CPU oracle for the NVFP4 KV-cache path. TEST INFRASTRUCTURE: only tests, the smoke check and the benchmark's CPU
baseline leg may import this package; the product package never does."""
