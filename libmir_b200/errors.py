"""Error types of the framework; every one carries a message that says what to fix."""


class LibmirError(Exception):
    """Base of every error the framework raises on purpose."""


class ConfigError(LibmirError):
    """config.json (or a runtime option) is missing a key, has a wrong type or an unsupported value."""


class RegistryError(LibmirError):
    """An architecture or a part kind is unknown to the registry."""


class WeightsError(LibmirError):
    """The checkpoint does not fit the model: lists missing, unexpected and wrongly shaped tensors."""

    def __init__(self, message, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)


class KernelError(LibmirError):
    """A kernel refuses its arguments (a size it does not take), or the native library is missing."""


class KvCapacity(LibmirError):
    """A request can never fit: it needs more pages than the whole pool holds (runtime/src/error.rs:24-27)."""

    def __init__(self, requested, capacity, group=""):
        super().__init__(f"request needs {requested} pages but the pool{' of ' + group if group else ''} holds {capacity}")
        self.requested, self.capacity = requested, capacity


class KvCachePressure(LibmirError):
    """Not enough free pages right now; pages come back when another request finishes."""

    def __init__(self, requested, free, group=""):
        super().__init__(f"need {requested} free pages{' in ' + group if group else ''}, only {free} are free")
        self.requested, self.free = requested, free


class NoFreeSlot(LibmirError):
    """Every per-request state slot is taken."""


class SchedulerError(LibmirError):
    """A request was submitted that the scheduler cannot run."""
