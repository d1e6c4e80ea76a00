"""Process-group plumbing: the CPU (gloo) backend and the single-GPU multi-rank emulation."""
