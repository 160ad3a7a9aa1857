"""Stand-in for hydra (absent offline): only `hydra.utils.instantiate` on plain dict configs."""
from . import utils  # noqa: F401


def main(*a, **k):
    def deco(fn):
        return fn
    return deco
