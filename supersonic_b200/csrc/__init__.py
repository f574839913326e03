"""Hand-written CUDA for sm_100a: sources, their build, and Python faces."""
