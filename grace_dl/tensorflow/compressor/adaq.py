from grace_b200.compressor.adaq import AdaqCompressor  # noqa: F401
