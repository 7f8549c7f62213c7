from grace_b200.compressor.qsgd import QSGDCompressor, QSGDCompressor_CUDA  # noqa: F401
