from grace_b200.compressor.fp16 import FP16Compressor  # noqa: F401
