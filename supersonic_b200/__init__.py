"""supersonic_b200: a small, whole generation library for one B200."""
__version__ = "0.1.0"
