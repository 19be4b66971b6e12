"""Small host-side helpers: synthetic streams, device timing, clock sampling, NVTX ranges."""
