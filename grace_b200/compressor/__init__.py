"""Compressors.  One module per algorithm, import paths mirror
``grace_dl/dist/compressor/*.py`` of the reference."""
from .none import NoneCompressor
from .fp16 import FP16Compressor
from .topk import TopKCompressor
from .randomk import RandomKCompressor
from .threshold import ThresholdCompressor
from .dgc import DgcCompressor
from .qsgd import QSGDCompressor, QSGDCompressor_CUDA
from .terngrad import TernGradCompressor
from .signsgd import SignSGDCompressor
from .signum import SignumCompressor
from .efsignsgd import EFSignSGDCompressor
from .onebit import OneBitCompressor
from .natural import NaturalCompressor, NaturalCompressor_CUDA
from .u8bit import U8bitCompressor
from .powersgd import PowerSGDCompressor
from .adaq import AdaqCompressor
from .sketch import SketchCompressor
from .inceptionn import INCEPTIONNCompressor

__all__ = [n for n in dir() if n.endswith("Compressor") or n.endswith("_CUDA")]
