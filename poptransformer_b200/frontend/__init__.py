"""GPU front end behind the reference's own graph-building API.

The reference never calls its native code directly: its model classes emit a PopART graph
(`popart.Builder`, `graph.aiOnnx.*`, `graph.aiGraphcore.*`, `graph.customOp(opName=...)`,
poptransformer/ops/popart.py:19-231 and ops/customized.py:21-148), `HFDecBaseModel.build_graph`
wraps the model graph into one Loop (models/base_model.py:271-290) and `Session.compile / run`
(sessions.py:35-49) hands it to `popart.InferenceSession`.  This package provides modules named
`popart` and `poprt` with that surface:

  * `popart.Builder` records the graph the unmodified model code emits;
  * `popart.InferenceSession.prepareDevice()` recognises the recorded decode loop (`lower.py`),
    takes the checkpoint out of the graph's initializers and builds the matching decoder of this
    package on the current CUDA device (Llama-2: the persistent step kernel or the per-op kernels);
  * `session.run(stepio)` feeds `input_ids`, runs the loop on the device and fills the anchors
    `Loop:0` (the id container) and `Loop:1` (the step) the reference reads back
    (models/llama2/model.py:218-230).

Use: put this directory first on PYTHONPATH (or call `install()`) before importing `poptransformer`,
and link `libpt_b200.so` as `custom_ops.so` where the reference loads it (ops/customized.py:17-18).
Nothing here runs on the CPU: a graph this front end does not recognise is refused at
`prepareDevice()`, like an op PopART cannot lower.
"""
import importlib
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def install():
    """Makes `import popart` / `import poprt` resolve to this package's modules."""
    if HERE not in sys.path:
        sys.path.insert(0, HERE)
    for name in ("popart", "poprt", "poprt.utils"):
        mod = sys.modules.get(name)
        if mod is not None and not getattr(mod, "__file__", "").startswith(HERE):
            del sys.modules[name]
    return importlib.import_module("popart")
