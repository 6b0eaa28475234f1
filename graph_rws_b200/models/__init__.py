from .model import GCN_BCSR  # noqa: F401
