"""ctypes wrapper of the C restatement (oracle/c/decode_ref.c): parity checker for larger shapes and
the timed CPU baseline.  Test infrastructure only."""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_build", "liboracle_ref.so")

c_void_p, c_int, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


class LayerStruct(ctypes.Structure):
    _fields_ = [("d_model", c_int), ("n_head", c_int), ("ffn", c_int), ("max_len", c_int), ("group", c_int), ("batch", c_int),
                ("eps", c_float)] + [(n, c_void_p) for n in (
                    "wq", "wk", "wv", "wo", "wgate", "wup", "wdown", "sq", "sk", "sv", "so", "sgate", "sup", "sdown",
                    "ln1", "ln2", "kcache", "vcache", "sin_t", "cos_t")]


def build():
    subprocess.run(["make", "-C", HERE], check=True, capture_output=True)
    return LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        _lib = ctypes.CDLL(LIB)
        _lib.oracle_llama_layer_step.argtypes = [ctypes.POINTER(LayerStruct), c_int, c_void_p, c_void_p]
        _lib.oracle_llama_head.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p]
        _lib.oracle_int4_linear.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
        _lib.oracle_f16_linear.argtypes = [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p]
    return _lib


def _p(a):
    return a.ctypes.data_as(c_void_p) if a is not None else None


def int4_linear(w, scale, x, group):
    n, k = w.shape[0], w.shape[1] * 2
    x = np.ascontiguousarray(x, dtype=np.float16)
    y = np.empty((x.shape[0], n), np.float16)
    lib().oracle_int4_linear(_p(np.ascontiguousarray(w)), _p(np.ascontiguousarray(scale, dtype=np.float16)), n, k, group, _p(x), x.shape[0], _p(y))
    return y


class LlamaOracleC:
    """Same interface as oracle.llama_np.LlamaOracle (tp = 1), running on the host cores."""

    def __init__(self, cfg, state_dict, batch, n_layer=None):
        from . import ops_np as O
        self.cfg, self.batch = cfg, batch
        c = cfg
        self.n_layer = c.n_layer if n_layer is None else n_layer
        self.sin, self.cos = O.llama_rope_tables(c.max_len, c.head_dim)
        self.keep = []   # numpy arrays referenced by the structs
        self.emb = np.ascontiguousarray(state_dict["model.embed_tokens.weight"], dtype=np.float16)
        self.layers = []
        names = [("wq", "self_attn.q_proj"), ("wk", "self_attn.k_proj"), ("wv", "self_attn.v_proj"), ("wo", "self_attn.o_proj"),
                 ("wgate", "mlp.gate_proj"), ("wup", "mlp.up_proj"), ("wdown", "mlp.down_proj")]
        for i in range(self.n_layer):
            p = f"model.layers.{i}."
            s = LayerStruct()
            s.d_model, s.n_head, s.ffn, s.max_len, s.group, s.batch, s.eps = c.d_model, c.n_head, c.ffn, c.max_len, c.group, batch, c.eps
            for f, nm in names:
                w = np.ascontiguousarray(state_dict[p + nm + ".weight"])
                self.keep.append(w)
                setattr(s, f, _p(w).value)
                if c.group:
                    sc = np.ascontiguousarray(state_dict[p + nm + ".weight_scale"], dtype=np.float16)
                    self.keep.append(sc)
                    setattr(s, "s" + f[1:], _p(sc).value)
            for f, nm in (("ln1", "input_layernorm.weight"), ("ln2", "post_attention_layernorm.weight")):
                a = np.ascontiguousarray(state_dict[p + nm], dtype=np.float16)
                self.keep.append(a)
                setattr(s, f, _p(a).value)
            kc = np.zeros((batch, c.n_head, c.max_len, c.head_dim), np.float16)
            vc = np.zeros_like(kc)
            self.keep += [kc, vc]
            s.kcache, s.vcache = _p(kc).value, _p(vc).value
            s.sin_t, s.cos_t = _p(self.sin).value, _p(self.cos).value
            self.layers.append(s)
        self.norm = np.ascontiguousarray(state_dict["model.norm.weight"], dtype=np.float16)
        self.head = np.ascontiguousarray(state_dict["lm_head.weight"], dtype=np.float16)
        self.scratch = np.empty(batch * (5 * c.d_model + 2 * c.ffn), np.float16)
        self.h = np.empty((batch, c.d_model), np.float16)
        self.lg = np.empty((batch, c.vocab), np.float16)
        self.nxt = np.empty(batch, np.int32)

    def _by_address(self, addr):
        return [a for a in self.keep if a.ctypes.data == addr][0]

    def kcache(self, layer):
        return self._by_address(self.layers[layer].kcache)

    def vcache(self, layer):
        return self._by_address(self.layers[layer].vcache)

    def set_cache(self, layer, k, v):
        """Loads a cache state: k, v [batch, n_head, max_len, head_dim] in the reference op's layout (newest token at index 0,
        zeros beyond the tokens cached so far), e.g. a paged cache exported with pt_kv_export."""
        self.kcache(layer)[...] = k
        self.vcache(layer)[...] = v

    def logits(self, ids_col, step):
        L = lib()
        x = np.ascontiguousarray(self.emb[np.asarray(ids_col).reshape(-1)])
        for s in self.layers:
            L.oracle_llama_layer_step(ctypes.byref(s), int(step), _p(x), _p(self.scratch))
        L.oracle_llama_head(_p(x), _p(self.norm), _p(self.head), self.batch, self.cfg.d_model, self.cfg.vocab, self.cfg.eps,
                            _p(self.h), _p(self.lg), _p(self.nxt))
        return self.lg.copy(), self.nxt.copy()
