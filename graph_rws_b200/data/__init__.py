from .bcsr import BCSRGraph  # noqa: F401
