from grace_b200.compressor.natural import NaturalCompressor  # noqa: F401
