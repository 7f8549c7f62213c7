from grace_b200.compressor.u8bit import U8bitCompressor  # noqa: F401
