"""Import-path compatibility package: ``grace_dl.dist`` and ``grace_dl.torch``
resolve to the implementations in ``grace_b200`` so that scripts written for
the reference run unchanged."""
__version__ = "1.0"
