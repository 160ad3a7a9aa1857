import importlib


def instantiate(cfg, **kwargs):
    if cfg is None:
        return None
    if isinstance(cfg, dict) and "_target_" in cfg:
        mod, _, name = cfg["_target_"].rpartition(".")
        cls = getattr(importlib.import_module(mod), name)
        args = {k: v for k, v in cfg.items() if k != "_target_"}
        args.update(kwargs)
        return cls(**args)
    return cfg
