"""poptransformer_b200: B200-native (sm_100a CUDA) backend for PopTransformer's per-token decode step.

The CUDA library is mandatory; importing the ops without it raises (no CPU fallback)."""
from ._lib import PtError  # noqa: F401
