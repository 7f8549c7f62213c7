from grace_b200.communicator.broadcast import Broadcast  # noqa: F401
