"""``grace_dl.tensorflow`` import path.

The reference's TensorFlow flavour builds graph-mode ops on ``tf.Tensor`` and rides on a patched Horovod
(``grace_dl/tensorflow/__init__.py:6-114``, ``patch_files/horovod/tensorflow``).  Neither TensorFlow nor Horovod
is part of this framework: the names below resolve to the PyTorch implementations in ``grace_b200`` (same
algorithms, same parameter names, ``torch.Tensor`` in and out), so that a script which only builds its
communicator through ``grace_from_params`` or the class constructors ports by changing its tensors, not its
configuration.  The four codecs that exist only in the reference's TensorFlow tree (AdaQ, INCEPTIONN, SketchML
quantile sketch, 8-bit) live here under their original module names.
"""
from grace_b200.core import Communicator, Compressor, Memory  # noqa: F401
