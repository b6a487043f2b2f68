"""bitnet.c_b200: a small B200-native library for Llama-style dense decoders."""
__version__ = "0.1.0"
