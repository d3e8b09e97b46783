"""Error types of the communication layer (reference: phyai/src/phyai/parallel/exceptions.py)."""


class PhyaiDistError(RuntimeError):
    """Base class for communication-layer failures."""


class NoBackendError(PhyaiDistError):
    """No registered backend can run the requested collective."""


class CommTimeoutError(PhyaiDistError):
    """A collective, a peer flag wait or a heartbeat ran out of time."""


class CaptureUnsafeError(PhyaiDistError):
    """A backend that cannot be captured in a CUDA graph was asked to run under capture."""


class PeerLostError(PhyaiDistError):
    """A rank stopped publishing heartbeats; the mesh must be rebuilt."""


__all__ = ["PhyaiDistError", "NoBackendError", "CommTimeoutError", "CaptureUnsafeError", "PeerLostError"]
