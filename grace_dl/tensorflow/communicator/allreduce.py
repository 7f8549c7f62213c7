from grace_b200.communicator.allreduce import Allreduce  # noqa: F401
