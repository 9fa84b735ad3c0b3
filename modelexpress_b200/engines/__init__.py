"""Engine adapters: the outermost drop-in seam (one module per engine)."""
