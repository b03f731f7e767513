from .bitlinear import BitLinear  # the reference exports exactly this (src/Metis/Metis/__init__.py:1)
