from .layer import BCSRGraphConv, BCSRSPMMFunction  # noqa: F401
