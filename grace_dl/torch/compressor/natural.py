from grace_b200.compressor.natural import NaturalCompressor, NaturalCompressor_CUDA  # noqa: F401
