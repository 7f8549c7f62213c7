from grace_b200.communicator.all_to_all import AllToAll  # noqa: F401
