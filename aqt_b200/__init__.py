"""B200-native quantized dot_general (the aqt.jax.v2 hot path) behind AQT's API."""

__version__ = '0.1.0'
