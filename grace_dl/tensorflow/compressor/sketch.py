from grace_b200.compressor.sketch import SketchCompressor  # noqa: F401
