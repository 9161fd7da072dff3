"""exo_b200: B200-native distributed inference (one process per GPU, NVLink collectives)."""
__version__ = "0.1.0"
