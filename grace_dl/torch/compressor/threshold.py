from grace_b200.compressor.threshold import ThresholdCompressor as _Threshold


class ThresholdCompressor(_Threshold):
    """Horovod flavour: keep ``|x| > threshold`` (``grace_dl/torch/compressor/threshold.py:17`` of the reference)."""

    def __init__(self, threshold):
        super().__init__(threshold, strict=True)
