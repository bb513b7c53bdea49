from .autocast_mode import autocast  # noqa: F401
