from grace_b200.communicator.allgather import Allgather  # noqa: F401
