"""A CPU stand-in for the `popart` Python module, just large enough to run the reference's UNMODIFIED graph-building
code (poptransformer/models, layers, ops) and execute the recorded graph with numpy.  TEST INFRASTRUCTURE ONLY: it is
used in the development container (where the reference tree is mounted) to produce golden vectors that pin the oracle.

Semantics: a Builder records nodes; `run_graph` interprets them.  Tensors are numpy arrays.  Every op on fp16 tensors is
computed in float32 and rounded once to fp16 (the oracle's definition of PopART/PopLibs fp16 arithmetic); matmul
accumulates in float32.  Custom ops dispatch to oracle/ops_np.py by the reference's op names.
"""
import contextlib
import math

import numpy as np

from oracle import ops_np as O

_DTYPES = {"FLOAT": np.float32, "FLOAT16": np.float16, "INT32": np.int32, "BOOL": np.bool_, "INT64": np.int64, "UINT8": np.uint8,
           "INT8": np.int8}


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
    OnePerGroup = "OnePerGroup"
    AllReplicas = "AllReplicas"


class CommGroupType:
    Consecutive, All, Orthogonal = "Consecutive", "All", "Orthogonal"


class CommGroup:
    def __init__(self, *a, **k):
        pass


class VariableSettings:
    def __init__(self, *a, **k):
        pass


class _Logger:
    def setLevel(self, level):
        pass


def getLogger(*a):
    return _Logger()


class _Node:
    __slots__ = ("op", "inputs", "outputs", "attrs", "state")

    def __init__(self, op, inputs, outputs, attrs):
        self.op, self.inputs, self.outputs, self.attrs, self.state = op, list(inputs), list(outputs), attrs, None


class _Namespace:
    """aiOnnx / aiGraphcore: every attribute is an op recorder."""

    def __init__(self, builder, domain):
        self._b, self._domain = builder, domain

    def __getattr__(self, op):
        def record(*args, **kwargs):
            return self._b._record(self._domain + "." + op, args, kwargs)
        return record


class Builder:
    def __init__(self, opsets=None, parent=None):
        self.parent = parent
        self.root = parent.root if parent else self
        self.nodes, self.inputs, self.outputs, self.initializers = [], [], [], {}
        self.parent_inputs = []
        self._scope = []
        self.aiOnnx = _Namespace(self, "onnx")
        self.aiGraphcore = _Namespace(self, "gc")
        if not parent:
            self._counter = 0
        self.name = "main"

    # ---- naming
    def _new_id(self, hint):
        self.root._counter += 1
        return f"{self.getNameScope()}{hint}:{self.root._counter}"      # popart prefixes ids with the name scope

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
    def _noop(self, *a, **k):
        yield

    virtualGraph = pipelineStage = outlineAttributes = _noop

    # ---- graph inputs / outputs
    def addInputTensor(self, info, *rest, debugContext=None):
        name = debugContext if debugContext is not None else (rest[-1] if rest and isinstance(rest[-1], str) else "input")
        tid = name if name not in self.inputs else self._new_id(name)
        self.inputs.append(tid)
        return tid

    def addUntypedInputTensor(self, name="input"):
        tid = self._new_id(name)
        self.inputs.append(tid)
        return tid

    def addInputTensorFromParentGraph(self, tensor_id):
        self.parent_inputs.append(tensor_id)
        self.inputs.append(tensor_id)

    def addInitializedInputTensor(self, array, *rest, debugContext=None):
        name = debugContext if debugContext is not None else (rest[-1] if rest and isinstance(rest[-1], str) else "init")
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
        return b""

    def saveInitializersExternally(self, *a, **k):
        pass

    def setAvailableMemoryProportion(self, *a, **k):
        pass

    setPartialsType = setSerializeMatMul = setAvailableMemoryProportion

    # ---- recording
    def _record(self, op, args, kwargs):
        kwargs = dict(kwargs)
        kwargs.pop("debugContext", None)
        inputs, attrs = [], kwargs
        if op == "onnx.constant":
            tid = self._new_id("const")
            node = _Node(op, [], [tid], {"value": np.asarray(args[0])})
            self.nodes.append(node)
            return tid
        if op == "onnx.loop":
            ins, n_out, body = args
            outs = [self._new_id("Loop") for _ in range(n_out)]
            # the reference reads anchors as 'Loop:0', 'Loop:1': keep those names for the first loop of the main graph
            outs = [f"Loop:{i}" for i in range(n_out)]
            self.nodes.append(_Node(op, ins, outs, {"body": body}))
            return outs
        if op == "onnx.randomnormal":
            tid = self._new_id("rand")
            self.nodes.append(_Node(op, [], [tid], attrs))
            return tid
        if args and isinstance(args[0], (list, tuple)):
            inputs = list(args[0])
            extra = args[1:]
        else:
            extra = args
        attrs["_extra"] = extra
        n_out = 1
        if op == "onnx.split":
            n_out = attrs["num_outputs"]
        elif op == "onnx.topk":
            n_out = 2
        elif op in ("gc.groupnormalization",):
            n_out = 3
        elif op == "gc.call":
            n_out = extra[0]
        outs = [self._new_id(op.split(".")[1]) for _ in range(n_out)]
        self.nodes.append(_Node(op, inputs, outs, attrs))
        if op in ("onnx.split", "onnx.topk", "gc.groupnormalization", "gc.call"):
            return outs
        return outs[0]

    def customOp(self, opName, opVersion=1, domain="ai.graphcore", inputs=(), attributes=None, numOutputs=1, **kw):
        outs = [self._new_id(opName) for _ in range(numOutputs)]
        self.nodes.append(_Node("custom." + opName, inputs, outs, dict(attributes or {})))
        return outs


# ------------------------------------------------------------------------------------------ interpreter
def _is16(*xs):
    return all(np.asarray(x).dtype == np.float16 for x in xs if np.asarray(x).dtype.kind == "f") and \
        any(np.asarray(x).dtype == np.float16 for x in xs)


def _fbin(fn, a, b):
    a, b = np.asarray(a), np.asarray(b)
    if a.dtype.kind == "f" or b.dtype.kind == "f":
        if _is16(a, b):
            return fn(a.astype(np.float32), b.astype(np.float32)).astype(np.float16)
        return fn(a.astype(np.float32), b.astype(np.float32)).astype(np.float32)
    return fn(a, b)


def _funary(fn, a):
    a = np.asarray(a)
    if a.dtype == np.float16:
        return fn(a.astype(np.float32)).astype(np.float16)
    return fn(a)


def _exec(node, env):
    op, a = node.op, node.attrs
    x = [env[i] for i in node.inputs]
    ex = a.get("_extra", ())
    if op == "onnx.constant":
        return [a["value"]]
    if op == "onnx.add":
        return [_fbin(np.add, *x)]
    if op == "onnx.sub":
        return [_fbin(np.subtract, *x)]
    if op == "onnx.mul":
        return [_fbin(np.multiply, *x)]
    if op == "onnx.div":
        return [_fbin(np.divide, *x)]
    if op == "onnx.matmul":
        p, q = np.asarray(x[0]), np.asarray(x[1])
        r = np.matmul(p.astype(np.float32), q.astype(np.float32))
        return [r.astype(np.float16) if _is16(p, q) else r]
    if op == "onnx.gather":
        return [np.take(x[0], np.asarray(x[1]).astype(np.int64), axis=a.get("axis", 0))]
    if op == "onnx.reshape":
        return [np.reshape(x[0], [int(v) for v in np.asarray(x[1]).reshape(-1)])]
    if op == "onnx.transpose":
        return [np.transpose(x[0], a["perm"])]
    if op == "onnx.split":
        idx = np.cumsum(a["split"])[:-1]
        return list(np.split(x[0], idx, axis=a["axis"]))
    if op == "onnx.concat":
        return [np.concatenate(x, axis=a["axis"])]
    if op == "onnx.cast":
        return [np.asarray(x[0]).astype(_DTYPES[ex[0]])]
    if op == "onnx.unsqueeze":
        r = np.asarray(x[0])
        for ax in sorted(ex[0] if ex else a["axes"]):
            r = np.expand_dims(r, ax)
        return [r]
    if op == "onnx.squeeze":
        return [np.squeeze(x[0], axis=tuple(ex[0] if ex else a["axes"]))]
    if op == "onnx.equal":
        return [np.equal(x[0], x[1])]
    if op == "onnx.less":
        return [np.less(x[0], x[1])]
    if op == "onnx.greater":
        return [np.greater(x[0], x[1])]
    if op == "onnx.where":
        return [np.where(np.asarray(x[0]).astype(bool), x[1], x[2])]
    if op == "onnx.topk":
        v, i = O.topk(np.asarray(x[0]), int(np.asarray(x[1]).reshape(-1)[0])) if a.get("axis", -1) in (-1, np.asarray(x[0]).ndim - 1) else (None, None)
        return [v, i]
    if op == "onnx.argmax":
        r = np.argmax(np.asarray(x[0]).astype(np.float32), axis=a["axis"])
        if a.get("keepdims", True):
            r = np.expand_dims(r, a["axis"])
        return [r.astype(np.int32)]
    if op == "onnx.reducemean":
        return [np.mean(np.asarray(x[0]), axis=tuple(a["axes"]), keepdims=bool(a.get("keepdims", 1)), dtype=np.asarray(x[0]).dtype)]
    if op == "onnx.reducesum":
        return [np.sum(x[0], axis=tuple(a["axes"]), keepdims=bool(a.get("keepdims", 1)))]
    if op == "onnx.sqrt":
        return [_funary(np.sqrt, x[0])]
    if op == "onnx.reciprocal":
        return [_funary(lambda v: np.float32(1.0) / v, x[0])]
    if op == "onnx.exp":
        return [_funary(np.exp, x[0])]
    if op == "onnx.sin":
        return [_funary(np.sin, x[0])]
    if op == "onnx.cos":
        return [_funary(np.cos, x[0])]
    if op == "onnx.tanh":
        return [_funary(np.tanh, x[0])]
    if op == "onnx.relu":
        return [np.maximum(x[0], 0)]
    if op == "onnx.sigmoid":
        return [O.sigmoid_f16(x[0]) if np.asarray(x[0]).dtype == np.float16 else 1 / (1 + np.exp(-x[0]))]
    if op == "onnx.softmax":
        return [O.softmax_v3(np.asarray(x[0]), True)]
    if op == "onnx.tile":
        return [np.tile(x[0], [int(v) for v in np.asarray(x[1])])]
    if op == "onnx.expand":
        # ONNX Expand: the result shape is the broadcast of the input shape with the requested shape
        return [np.broadcast_to(x[0], np.broadcast_shapes(np.shape(x[0]), tuple(int(v) for v in np.asarray(x[1])))).copy()]
    if op == "gc.swish":
        return [O.swish_f16(x[0])]
    if op == "gc.gelu":
        return [O.gelu_f16(x[0])]
    if op == "gc.bitwiseor":
        return [np.bitwise_or(x[0], x[1])]
    if op == "gc.bitwiseand":
        return [np.bitwise_and(x[0], x[1])]
    if op == "gc.slice":
        sl = [slice(None)] * np.asarray(x[0]).ndim
        for s, e, ax in zip(a["starts"], a["ends"], a["axes"]):
            sl[ax] = slice(s, e)
        return [np.asarray(x[0])[tuple(sl)]]
    if op == "gc.dynamicslice":
        idx = int(np.asarray(x[1]).reshape(-1)[0])
        sl = [slice(None)] * np.asarray(x[0]).ndim
        sl[a["axes"][0]] = slice(idx, idx + a["sizes"][0])
        r = np.asarray(x[0])[tuple(sl)]
        if r.shape[a["axes"][0]] != a["sizes"][0]:
            raise IndexError("dynamicslice out of range (run max_loop <= max_length - 1 iterations)")
        return [r]
    if op == "gc.dynamicupdate":
        idx = int(np.asarray(x[1]).reshape(-1)[0])
        r = np.array(x[0], copy=True)
        sl = [slice(None)] * r.ndim
        sl[a["axes"][0]] = slice(idx, idx + a["sizes"][0])
        r[tuple(sl)] = np.asarray(x[2]).reshape(r[tuple(sl)].shape)
        return [r]
    if op == "gc.replicatedallreduce":
        return [x[0]]
    if op == "gc.printtensor":
        return [x[0]]
    if op == "custom.KVCache":
        if node.state is None:
            node.state = O.KVCacheState()
        return [O.kv_cache(node.state, int(np.asarray(x[0]).reshape(-1)[0]), x[1], a["max_len"], a["sequence_axis"], a["step_len"])]
    if op == "custom.SoftmaxV3":
        return [O.softmax_v3(np.asarray(x[0]), bool(a["stable_mode"]))]
    if op == "custom.NormCE":
        return [O.norm_ce(x[0], x[1], x[2], a["epsilon"])]
    if op == "custom.Int4ToHalf":
        return [O.int4_to_half(x[0], x[1], axis=a["axis"])]
    if op == "custom.Remap":
        return [x[0]]
    raise NotImplementedError(op)


def run_graph(builder, feeds, parent_env=None):
    """Executes the recorded graph; returns the environment (tensor id -> array)."""
    env = dict(parent_env or {})
    env.update(builder.initializers)
    env.update(feeds)
    for node in builder.nodes:
        if node.op == "onnx.loop":
            body = node.attrs["body"]
            max_loop = int(np.asarray(env[node.inputs[0]]))
            carried = [env[i] for i in node.inputs[2:]]
            cond = bool(np.asarray(env[node.inputs[1]]))
            body_in = body.inputs            # ['max_loop', 'cond', carried...]
            it = 0
            while it < max_loop and cond:
                feeds_b = {body_in[0]: np.int32(it), body_in[1]: np.bool_(cond)}
                feeds_b.update({tid: v for tid, v in zip(body_in[2:], carried)})
                benv = run_graph(body, feeds_b, parent_env=env)
                outs = [benv[t] for t in body.outputs]
                cond = bool(np.asarray(outs[0]))
                carried = outs[1:]
                it += 1
            for tid, v in zip(node.outputs, carried):
                env[tid] = v
            continue
        outs = _exec(node, env)
        for tid, v in zip(node.outputs, outs):
            env[tid] = v
    return env
