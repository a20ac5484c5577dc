"""Hand-written sm_100a kernels: sources in `csrc/`, Python entry points in `ops`."""
