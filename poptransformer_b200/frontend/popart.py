"""`popart`-compatible recorder and session for the B200 backend (see the package docstring).

Only what the reference's decode models touch is provided (sessions.py, models/base_model.py:116-131, layers/base_layer.py,
utils/registry.py): Builder with its aiOnnx / aiGraphcore namespaces and customOp, the value classes the model code passes
around, and InferenceSession / PyStepIO / DataFlow / DeviceManager / SessionOptions.  Recording keeps op names, attributes and
constant values; nothing is computed at record time."""
import contextlib
import json

import numpy as np

__version__ = "poptransformer_b200 front end"


class TensorInfo:
    def __init__(self, dtype, shape):
        self.dtype, self.shape = dtype, list(shape)


class InputSettings:
    def __init__(self, *a, **k):
        pass


class ReplicatedStreamMode:
    Broadcast = "Broadcast"


class AnchorReturnType:
    def __init__(self, name):
        self.name = name


class VariableRetrievalMode:
    OnePerGroup, AllReplicas = "OnePerGroup", "AllReplicas"


class CommGroupType:
    Consecutive, All, Orthogonal, Ungrouped = "Consecutive", "All", "Orthogonal", "None"


class CommGroup:
    def __init__(self, *a, **k):
        self.args, self.kwargs = a, k


class VariableSettings:
    def __init__(self, *a, **k):
        self.args, self.kwargs = a, k


class VirtualGraphMode:
    Off, Manual, Auto = "Off", "Manual", "Auto"


class SessionOptions:
    """Attribute bag: the reference sets IPU compilation switches (sessions.py:62-90) that have no meaning here."""


class DataFlow:
    def __init__(self, batches_per_step, anchors):
        self.batches_per_step, self.anchors = batches_per_step, dict(anchors)


class _Device:
    def __init__(self, n):
        self.numIpus = n


class DeviceManager:
    def acquireAvailableDevice(self, n=1, *a, **k):
        return _Device(n)

    createIpuModelDevice = createCpuDevice = acquireAvailableDevice


class PyStepIO:
    def __init__(self, inputs, outputs):
        self.inputs, self.outputs = inputs, outputs


class _Logger:
    def setLevel(self, level):
        pass


def getLogger(*a):
    return _Logger()


class Node:
    __slots__ = ("op", "inputs", "outputs", "attrs")

    def __init__(self, op, inputs, outputs, attrs):
        self.op, self.inputs, self.outputs, self.attrs = op, list(inputs), list(outputs), attrs


class _Namespace:
    """aiOnnx / aiGraphcore: every attribute records an op of that name."""

    def __init__(self, builder, domain):
        self._b, self._domain = builder, domain

    def __getattr__(self, op):
        def record(*args, **kwargs):
            return self._b._record(self._domain + "." + op, args, kwargs)
        return record


_MULTI_OUT = {"onnx.topk": 2, "gc.groupnormalization": 3}


class Builder:
    def __init__(self, opsets=None, parent=None):
        self.parent = parent
        self.root = parent.root if parent else self
        self.nodes, self.inputs, self.outputs, self.initializers = [], [], [], {}
        self.input_info = {}       # shape and dtype of the inputs that were declared with a TensorInfo
        self._scope = []
        self.aiOnnx = _Namespace(self, "onnx")
        self.aiGraphcore = _Namespace(self, "gc")
        if not parent:
            self._counter = 0
        self.name = "main"

    # ---- naming (PopART prefixes tensor ids with the name scope)
    def _new_id(self, hint):
        self.root._counter += 1
        return f"{self.getNameScope()}{hint}:{self.root._counter}"

    @contextlib.contextmanager
    def nameScope(self, name):
        self._scope.append(str(name))
        try:
            yield
        finally:
            self._scope.pop()

    def getNameScope(self):
        return "/".join(self._scope) + ("/" if self._scope else "")

    @contextlib.contextmanager
    def _placement(self, *a, **k):    # IPU placement / outlining hints
        yield

    virtualGraph = pipelineStage = outlineAttributes = executionPhase = _placement

    # ---- graph inputs / outputs
    @staticmethod
    def _name(rest, debug, default):
        if debug is not None:
            return debug
        return rest[-1] if rest and isinstance(rest[-1], str) else default

    def addInputTensor(self, info, *rest, debugContext=None):
        name = self._name(rest, debugContext, "input")
        tid = name if name not in self.inputs else self._new_id(name)
        self.inputs.append(tid)
        if isinstance(info, TensorInfo):
            self.input_info[tid] = {"shape": [int(v) for v in info.shape], "dtype": str(info.dtype)}
        return tid

    def addUntypedInputTensor(self, name="input"):
        tid = self._new_id(name)
        self.inputs.append(tid)
        return tid

    def addInputTensorFromParentGraph(self, tensor_id):
        self.inputs.append(tensor_id)

    def addInitializedInputTensor(self, array, *rest, debugContext=None):
        name = self._name(rest, debugContext, "init")
        tid = name if name not in self.initializers else self._new_id(name)
        self.initializers[tid] = np.asarray(array)
        self.inputs.append(tid)
        return tid

    def addOutputTensor(self, tensor_id):
        self.outputs.append(tensor_id)

    def getInputTensorIds(self):
        return list(self.inputs)

    def getOutputTensorIds(self):
        return list(self.outputs)

    def isInitializer(self, tensor_id):
        return tensor_id in self.initializers

    def createSubgraphBuilder(self):
        return Builder(parent=self)

    def setGraphName(self, name):
        self.name = name

    def getModelProto(self):
        return RecordedModel(self.root)

    def saveInitializersExternally(self, *a, **k):
        pass

    def setAvailableMemoryProportion(self, *a, **k):
        pass

    setPartialsType = setSerializeMatMul = recomputeOutputInBackwardPass = setAvailableMemoryProportion

    # ---- recording
    def _record(self, op, args, kwargs):
        attrs = dict(kwargs)
        attrs.pop("debugContext", None)
        if op == "onnx.constant":
            tid = self._new_id("const")
            self.nodes.append(Node(op, [], [tid], {"value": np.asarray(args[0])}))
            return tid
        if op == "onnx.loop":
            ins, n_out, body = args
            outs = [f"Loop:{i}" for i in range(n_out)]     # the ids the reference reads its anchors by (llama2/model.py:218-230)
            self.nodes.append(Node(op, ins, outs, {"body": body}))
            return outs
        if args and isinstance(args[0], (list, tuple)):
            inputs, extra = list(args[0]), list(args[1:])
        else:
            inputs, extra = [], list(args)
        attrs["_extra"] = extra
        n_out = _MULTI_OUT.get(op, 1)
        if op == "onnx.split":
            n_out = attrs["num_outputs"]
        elif op == "gc.call":
            n_out = extra[0]
        outs = [self._new_id(op.split(".")[1]) for _ in range(n_out)]
        self.nodes.append(Node(op, inputs, outs, attrs))
        return outs if n_out > 1 or op in ("onnx.split", "gc.call") else outs[0]

    def customOp(self, opName, opVersion=1, domain="ai.graphcore", inputs=(), attributes=None, numOutputs=1, **kw):
        outs = [self._new_id(opName) for _ in range(numOutputs)]
        self.nodes.append(Node("custom." + opName, inputs, outs, dict(attributes or {})))
        return outs

    # ---- (de)serialisation of a recorded graph without its weights: what a test on a machine without the reference loads
    def to_dict(self):
        def enc(v):
            if isinstance(v, Builder):
                return {"__graph__": v.to_dict()}
            if isinstance(v, np.ndarray) or isinstance(v, np.generic):
                a = np.asarray(v)
                return {"__array__": a.tolist(), "dtype": str(a.dtype)}
            if isinstance(v, (list, tuple)):
                return [enc(x) for x in v]
            return v
        return {"name": self.name, "inputs": self.inputs, "outputs": self.outputs, "input_info": self.input_info,
                "initializers": {k: {"shape": list(v.shape), "dtype": str(v.dtype)} for k, v in self.initializers.items()},
                "nodes": [{"op": n.op, "inputs": n.inputs, "outputs": n.outputs, "attrs": {k: enc(v) for k, v in n.attrs.items()}} for n in self.nodes]}

    @classmethod
    def from_dict(cls, d, parent=None):
        b = cls(parent=parent)
        b.name, b.inputs, b.outputs = d["name"], list(d["inputs"]), list(d["outputs"])
        b.input_info = dict(d.get("input_info", {}))
        b.initializers = {k: None for k in d["initializers"]}     # arrays are attached by the caller
        b.initializer_info = d["initializers"]

        def dec(v):
            if isinstance(v, dict) and "__graph__" in v:
                return cls.from_dict(v["__graph__"], parent=b)
            if isinstance(v, dict) and "__array__" in v:
                return np.asarray(v["__array__"], dtype=v["dtype"])
            if isinstance(v, list):
                return [dec(x) for x in v]
            return v
        b.nodes = [Node(n["op"], n["inputs"], n["outputs"], {k: dec(v) for k, v in n["attrs"].items()}) for n in d["nodes"]]
        return b

    def save(self, path):
        with open(path, "w") as f:
            json.dump(self.to_dict(), f)

    @classmethod
    def load(cls, path):
        with open(path) as f:
            return cls.from_dict(json.load(f))


class RecordedModel:
    """What `Builder.getModelProto()` hands to InferenceSession in place of a serialised ONNX model."""

    def __init__(self, builder):
        self.builder = builder


class InferenceSession:
    """popart.InferenceSession for the recorded decode graphs (sessions.py:92-100, 35-49)."""

    def __init__(self, fnModel, dataFlow=None, deviceInfo=None, userOptions=None, **kw):
        self.builder = fnModel.builder if isinstance(fnModel, RecordedModel) else fnModel
        if not isinstance(self.builder, Builder):
            raise TypeError("InferenceSession needs the model recorded by this module's Builder (graph.getModelProto())")
        self.data_flow, self.options = dataFlow, userOptions
        self.decoder = self.plan = None
        self.decoder_kwargs = {}

    def prepareDevice(self, *a, **k):
        self.plan, self.decoder = _lower_entry(self.builder, **self.decoder_kwargs)

    def weightsFromHost(self):
        pass    # the decoder packed the checkpoint into device memory when it was built

    def initAnchorArrays(self):
        p = self.plan
        self.anchors = {"Loop:0": np.zeros((p.batch, p.max_len), np.int32), "Loop:1": np.zeros((), np.int32)}
        if self.data_flow is not None:
            for name in self.data_flow.anchors:
                self.anchors.setdefault(name, np.zeros((), np.int32))
        return self.anchors

    def run(self, stepio):
        if self.decoder is None:
            raise RuntimeError("InferenceSession.run before prepareDevice")
        ids = np.asarray(stepio.inputs["input_ids"], dtype=np.int32).reshape(self.plan.batch, self.plan.max_len)
        out = self.decoder.run(ids, max_loop=self.plan.max_loop)
        np.copyto(stepio.outputs["Loop:0"], out["Loop:0"])
        np.copyto(stepio.outputs["Loop:1"], np.asarray(out["Loop:1"]).reshape(()))


def _lower_entry(builder, **kw):
    import importlib
    import os
    import sys
    pkg_parent = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    if pkg_parent not in sys.path:
        sys.path.insert(0, pkg_parent)
    lower = importlib.import_module("poptransformer_b200.frontend.lower")
    return lower.lower(builder, **kw)
