"""Performance drivers equivalent to the reference's perftest/ tree (run them under torchrun)."""
