"""Stand-in for the un-vendored `poprt` wheel (only what poptransformer imports)."""
from . import utils  # noqa: F401
