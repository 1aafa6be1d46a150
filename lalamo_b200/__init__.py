"""A B200-native inference engine for the LFM2 architecture."""

__version__ = "0.1.0"
