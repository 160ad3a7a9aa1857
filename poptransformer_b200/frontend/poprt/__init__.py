"""Stand-in for the `poprt` wheel the reference imports (utils/param_handler/precision_strategy.py:15): only its
FP8 converter is used, and only by the Graphcore-FP8 precision modes, which this backend replaces by OCP E4M3."""
from . import utils  # noqa: F401
