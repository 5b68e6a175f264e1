"""A B200-native inference engine for Gemma 1: from a model folder to generated tokens on one GPU."""
__version__ = "0.1.0"
