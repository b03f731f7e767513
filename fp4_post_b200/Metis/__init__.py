"""Host-side mirror of the reference's `src/Metis` package (only what the NVFP4 linear path needs)."""
