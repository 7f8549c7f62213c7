from grace_b200.compressor.efsignsgd import EFSignSGDCompressor  # noqa: F401
