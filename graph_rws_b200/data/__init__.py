from .bcsr import BCSRGraph  # noqa: F401
from .bcsr_io import bcsr_bin_paths, load_bcsr_bins, save_bcsr_bins  # noqa: F401
from .topology import CSRTopology  # noqa: F401
