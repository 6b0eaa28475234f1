"""graph_rws_b200: the BCSR SpMM and neighbour-sampling hot path of Graph_RWS, rebuilt for B200.

Sub-packages mirror the reference's layout for the parts on the path:
core (operators over the C ABI), data (BCSRGraph), layers, models, sampler, helper.
"""
from .data import BCSRGraph  # noqa: F401
from .layers import BCSRGraphConv, BCSRSPMMFunction  # noqa: F401
from .models import GCN_BCSR  # noqa: F401

__version__ = "0.1.0"
