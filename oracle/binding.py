"""TEST INFRASTRUCTURE ONLY: ctypes bindings for the two CPU checkers.

`Port`  -> oracle/liboracle_port.so   (our restatement, port.cpp, prefix ``orp_``)
`Ref`   -> oracle/_ref/libsfref.so    (the unmodified reference sources behind
                                       ref_harness.cpp, prefix ``sfref_``)

Both expose the same Python methods so that a test can run the same call against
either.  Nothing under the product package may import this module; only tests/,
the smoke check and bench.py's CPU-baseline legs do.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "liboracle_port.so")
REF_SO = os.path.join(HERE, "_ref", "libsfref.so")

f32p = C.POINTER(C.c_float)
i32p = C.POINTER(C.c_int)


class DecoderConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("batch", "sequence", "hidden", "intermediate",
                                       "query_heads", "kv_heads", "head_dim")] + \
               [("rms_epsilon", C.c_float), ("rope_theta", C.c_float)] + \
               [(n, C.c_int) for n in ("causal", "ffn_moe", "experts", "top_k", "context_sequence")]


DATA_FIELDS = ("input", "rms1_weight", "query_weight", "key_weight", "value_weight",
               "output_weight", "rms2_weight", "gate_weight", "up_weight", "down_weight",
               "router_weight", "w1", "w3", "w2", "cached_key", "cached_value")


class DecoderData(C.Structure):
    _fields_ = [(n, f32p) for n in DATA_FIELDS] + \
               [("trace_expert_ids", i32p), ("trace_expert_weights", f32p), ("trace_counts", i32p)]


class AttentionConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("batch", "query_heads", "kv_heads", "sequence_query",
                                       "sequence_kv", "head_dim", "head_dim_value", "causal")] + \
               [("scale", C.c_float)]


class MoeConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("tokens", "hidden", "intermediate", "experts", "top_k")]


def fp(a):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(f32p)


def ip(a):
    if a is None:
        return None
    assert a.dtype == np.int32 and a.flags.c_contiguous
    return a.ctypes.data_as(i32p)


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def decoder_config(batch=1, sequence=16, hidden=64, intermediate=128, query_heads=4, kv_heads=2,
                   head_dim=16, rms_epsilon=1e-5, rope_theta=10000.0, causal=True, moe=False,
                   experts=4, top_k=2, context_sequence=0):
    return DecoderConfig(batch, sequence, hidden, intermediate, query_heads, kv_heads, head_dim,
                         rms_epsilon, rope_theta, int(causal), int(moe), experts, top_k,
                         context_sequence)


INT8_WEIGHTS = {"query_weight": ("hidden", "hidden"), "key_weight": ("hidden", "kv"), "value_weight": ("hidden", "kv"),
                "output_weight": ("hidden", "hidden"), "gate_weight": ("hidden", "intermediate"),
                "up_weight": ("hidden", "intermediate"), "down_weight": ("intermediate", "hidden")}


def quantize_dequantize(w_in_out):
    """quantize_matmul_weights (src/next_milestones.cpp:611-637) per output channel of an [in, out]
    weight, then q * scale again: the weights the reference's INT8 layer effectively multiplies by."""
    w = np.asarray(w_in_out, np.float32)
    maximum = np.max(np.abs(w), axis=0)
    scale = np.where(maximum > 0, (maximum / np.float32(127.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)
    value = (w / scale[None, :]).astype(np.float32)
    q = np.clip(np.sign(value) * np.floor(np.abs(value) + np.float32(0.5)), -127, 127).astype(np.float32)
    return (q * scale[None, :]).astype(np.float32)


def int8_expert_weights(w, experts, rows, cols):
    """Expert weights [experts, rows(in), cols(out)] after the INT8 round trip of quantize_moe_weights
    (src/next_milestones.cpp:699-714): every expert matrix on its own, per output channel."""
    w = np.asarray(w, np.float32).reshape(experts, rows, cols)
    return np.stack([quantize_dequantize(w[e]) for e in range(experts)]).reshape(-1)


def int8_weight_data(c, data):
    """DecoderData with the seven dense weights replaced by their INT8 round trip."""
    dims = {"hidden": c.hidden, "kv": c.kv_heads * c.head_dim, "intermediate": c.intermediate}
    out = dict(data)
    for name, (rows, cols) in INT8_WEIGHTS.items():
        out[name] = quantize_dequantize(np.asarray(data[name], np.float32).reshape(dims[rows], dims[cols])).reshape(-1)
    return out


def decoder_shapes(c):
    """Element counts of every DecoderData tensor for configuration `c`."""
    t, h, i = c.batch * c.sequence, c.hidden, c.intermediate
    kv = c.kv_heads * c.head_dim
    s = {"input": t * h, "rms1_weight": h, "query_weight": h * h, "key_weight": h * kv,
         "value_weight": h * kv, "output_weight": h * h, "rms2_weight": h}
    if c.ffn_moe:
        s.update(router_weight=h * c.experts, w1=c.experts * h * i, w3=c.experts * h * i,
                 w2=c.experts * i * h)
    else:
        s.update(gate_weight=h * i, up_weight=h * i, down_weight=i * h)
    if c.context_sequence > 0:
        n = c.batch * c.kv_heads * c.context_sequence * c.head_dim
        s.update(cached_key=n, cached_value=n)
    return s


def pack_decoder_data(data, trace=None):
    """dict of float32 arrays -> (DecoderData struct, keepalive list)."""
    keep = {k: f32(v) for k, v in data.items() if v is not None}
    d = DecoderData()
    for name in DATA_FIELDS:
        setattr(d, name, fp(keep.get(name)))
    if trace is not None:
        ids, weights, counts = i32(trace[0]), f32(trace[1]), i32(trace[2])
        keep["_trace"] = (ids, weights, counts)
        d.trace_expert_ids, d.trace_expert_weights, d.trace_counts = ip(ids), fp(weights), ip(counts)
    return d, keep


def build(which="all"):
    """Compile the checkers (the reference one only where the reference source tree is present)."""
    targets = []
    if which in ("all", "port"):
        targets.append("port")
    if which in ("all", "ref") and os.path.isdir(os.environ.get("SFB_REFERENCE", "/root/reference")):
        targets.append("ref")
    for target in targets:
        subprocess.run(["make", "-C", HERE, target, "-j8",
                        "REF=" + os.environ.get("SFB_REFERENCE", "/root/reference")],
                       check=True, stdout=subprocess.DEVNULL)


class OracleError(RuntimeError):
    def __init__(self, code, message=""):
        super().__init__(f"oracle status {code}: {message}")
        self.code = code


class _Base:
    prefix = ""

    def __init__(self, path):
        self.lib = C.CDLL(path)
        self.path = path

    def fn(self, name, restype=C.c_int):
        f = getattr(self.lib, self.prefix + name)
        f.restype = restype
        return f

    def hardware_threads(self):
        return self.fn("hardware_threads")()


class Port(_Base):
    """Our restatement (oracle/port.cpp)."""
    prefix = "orp_"
    kind = "port"

    def __init__(self):
        if not os.path.exists(PORT_SO):
            build("port")
        super().__init__(PORT_SO)

    def round_bf16(self, a):
        a = f32(a).copy()
        self.fn("round_bf16", None)(fp(a), C.c_longlong(a.size))
        return a

    def rms_norm(self, x, w, eps):
        x, w = f32(x), f32(w)
        out = np.empty_like(x)
        self.fn("rms_norm", None)(fp(x), fp(w), x.shape[0], x.shape[1], C.c_float(eps), fp(out))
        return out

    def matmul(self, a, b, fma=False, threads=0):
        a, b = f32(a), f32(b)
        c = np.empty((a.shape[0], b.shape[1]), np.float32)
        self.fn("matmul", None)(fp(a), fp(b), fp(c), a.shape[0], b.shape[1], a.shape[1],
                                int(fma), threads)
        return c

    def split_qkv_rope(self, c, fused):
        fused = f32(fused)
        q = np.empty((c.batch, c.query_heads, c.sequence, c.head_dim), np.float32)
        k = np.empty((c.batch, c.kv_heads, c.sequence, c.head_dim), np.float32)
        v = np.empty_like(k)
        self.fn("split_qkv_rope", None)(C.byref(c), fp(fused), fp(q), fp(k), fp(v))
        return q, k, v

    def swiglu(self, gate_up, intermediate):
        gate_up = f32(gate_up)
        out = np.empty((gate_up.shape[0], intermediate), np.float32)
        self.fn("swiglu", None)(fp(gate_up), gate_up.shape[0], intermediate, fp(out))
        return out

    def _attn_out(self, c):
        return np.empty((c.batch, c.query_heads, c.sequence_query, c.head_dim_value), np.float32)

    def attention_reference(self, c, q, k, v, threads=0):
        q, k, v = f32(q), f32(k), f32(v)
        out = self._attn_out(c)
        self.fn("attention_reference", None)(C.byref(c), fp(q), fp(k), fp(v), fp(out), threads)
        return out

    def attention_materialized(self, c, q, k, v):
        q, k, v = f32(q), f32(k), f32(v)
        out = self._attn_out(c)
        self.fn("attention_materialized", None)(C.byref(c), fp(q), fp(k), fp(v), fp(out))
        return out

    def attention_io_aware(self, c, q, k, v, query_tile, kv_tile, threads=0):
        q, k, v = f32(q), f32(k), f32(v)
        out = self._attn_out(c)
        self.fn("attention_io_aware", None)(C.byref(c), query_tile, kv_tile, fp(q), fp(k), fp(v),
                                            fp(out), threads)
        return out

    def attention_split_kv(self, c, q, k, v, splits, kv_tile=64, threads=0):
        q, k, v = f32(q), f32(k), f32(v)
        out = self._attn_out(c)
        self.fn("attention_split_kv", None)(C.byref(c), splits, kv_tile, fp(q), fp(k), fp(v),
                                            fp(out), threads)
        return out

    # paged KV --------------------------------------------------------------------
    def paged_create(self, batch, kv_heads, dim, dim_v, page_tokens, capacity):
        h = self.fn("paged_create", C.c_void_p)(batch, kv_heads, dim, dim_v, page_tokens, capacity)
        if not h:
            raise OracleError(1, "invalid paged KV configuration")
        return PagedHandle(self, h, (batch, kv_heads, dim, dim_v, page_tokens, capacity))

    # MoE -------------------------------------------------------------------------
    def route_topk(self, c, x, router_weight, bias=None):
        x, router_weight = f32(x), f32(router_weight)
        tokens = x.shape[0]
        ids = np.empty((tokens, c.top_k), np.int32)
        weights = np.empty((tokens, c.top_k), np.float32)
        counts = np.empty(c.experts, np.int32)
        ties = C.c_int(0)
        b = f32(bias) if bias is not None else None
        self.fn("route_topk", None)(C.byref(c), fp(x), tokens, fp(router_weight), fp(b), ip(ids),
                                    fp(weights), ip(counts), C.byref(ties))
        self.last_tie_tokens = ties.value
        return ids, weights, counts

    def dispatch_tokens(self, c, x, ids, weights, counts, copy_values=True):
        x, ids, weights, counts = f32(x), i32(ids), f32(weights), i32(counts)
        tokens = ids.shape[0]
        n = tokens * c.top_k
        values = np.empty((n, c.hidden), np.float32) if copy_values else None
        offsets = np.empty(c.experts + 1, np.int32)
        token_ids, slots = np.empty(n, np.int32), np.empty(n, np.int32)
        rw = np.empty(n, np.float32)
        self.fn("dispatch_tokens", None)(C.byref(c), fp(x), tokens, ip(ids), fp(weights),
                                         ip(counts), fp(values), ip(offsets), ip(token_ids),
                                         ip(slots), fp(rw))
        return values, offsets, token_ids, slots, rw

    def plan_moe_tasks(self, c, counts, split_threshold=0):
        counts = i32(counts)
        tasks = np.empty((4096, 4), np.int32)
        n = self.fn("plan_moe_tasks")(C.byref(c), ip(counts), split_threshold, ip(tasks), 4096)
        return tasks[:n].copy()

    def moe_reference(self, c, x, w1, w3, w2, ids, weights, threads=0):
        x, w1, w3, w2, ids, weights = f32(x), f32(w1), f32(w3), f32(w2), i32(ids), f32(weights)
        out = np.empty((x.shape[0], c.hidden), np.float32)
        self.fn("moe_reference", None)(C.byref(c), fp(x), x.shape[0], fp(w1), fp(w3), fp(w2),
                                       ip(ids), fp(weights), fp(out), threads)
        return out

    def moe_grouped(self, c, x, w1, w3, w2, ids, weights, counts, threads=0):
        x, w1, w3, w2 = f32(x), f32(w1), f32(w3), f32(w2)
        ids, weights, counts = i32(ids), f32(weights), i32(counts)
        out = np.empty((x.shape[0], c.hidden), np.float32)
        self.fn("moe_grouped", None)(C.byref(c), fp(x), x.shape[0], fp(w1), fp(w3), fp(w2),
                                     ip(ids), fp(weights), ip(counts), fp(out), threads)
        return out

    def decoder_layer(self, c, data, native=False, threads=0, trace=None, want_normalized2=False):
        d, keep = pack_decoder_data(data, trace)
        t = c.batch * c.sequence
        out = np.empty((t, c.hidden), np.float32)
        n2 = np.empty((t, c.hidden), np.float32) if want_normalized2 else None
        self.fn("decoder_layer", None)(C.byref(c), C.byref(d), int(native), threads, fp(out), fp(n2))
        del keep
        return (out, n2) if want_normalized2 else out


class PagedHandle:
    """Paged KV cache living inside one of the checkers."""

    def __init__(self, owner, handle, config):
        self.o, self.h, self.config = owner, C.c_void_p(handle), config

    def _check(self, status):
        if status != 0:
            msg = self.o.fn("last_error", C.c_char_p)().decode() if self.o.prefix == "sfref_" else ""
            raise OracleError(status, msg)

    def set_free_pages(self, pages):
        pages = i32(pages)
        r = self.o.fn("paged_set_free_pages", C.c_int if self.o.prefix == "sfref_" else None)(
            self.h, ip(pages), pages.size)
        if self.o.prefix == "sfref_":
            self._check(r)

    def append(self, keys, values, tokens):
        keys, values = f32(keys), f32(values)
        self._check(self.o.fn("paged_append")(self.h, fp(keys), fp(values), tokens))

    def truncate(self, n):
        self._check(self.o.fn("paged_truncate")(self.h, n))

    def release(self, pages):
        pages = i32(pages)
        self._check(self.o.fn("paged_release")(self.h, ip(pages), pages.size))

    def info(self):
        info = np.zeros(4, np.int32)
        table, free = np.zeros(65536, np.int32), np.zeros(65536, np.int32)
        self.o.fn("paged_info", None if self.o.prefix == "orp_" else C.c_int)(
            self.h, ip(info), ip(table), table.size, ip(free), free.size)
        return {"length": int(info[0]), "page_table": table[:info[1]].copy(),
                "free_pages": free[:info[2]].copy(), "pages": int(info[3])}

    def storage(self):
        b, hkv, d, dv, p, cap = self.config
        pages = (cap + p - 1) // p
        keys = np.empty((pages, b, hkv, p, d), np.float32)
        values = np.empty((pages, b, hkv, p, dv), np.float32)
        self.o.fn("paged_storage", None if self.o.prefix == "orp_" else C.c_int)(
            self.h, fp(keys), fp(values))
        return keys, values

    def gather(self):
        b, hkv, d, dv, _, _ = self.config
        n = self.info()["length"]
        keys = np.empty((b, hkv, max(n, 0), d), np.float32)
        values = np.empty((b, hkv, max(n, 0), dv), np.float32)
        self._check(self.o.fn("paged_gather")(self.h, fp(keys), fp(values)))
        return keys, values

    def decode(self, c, query, two_pass=False):
        query = f32(query)
        out = np.empty((c.batch, c.query_heads, c.sequence_query, c.head_dim_value), np.float32)
        if self.o.prefix == "orp_":
            self._check(self.o.fn("paged_decode")(self.h, C.byref(c), fp(query), fp(out),
                                                  int(two_pass)))
        else:
            err = C.c_double(0)
            self._check(self.o.fn("paged_decode")(self.h, C.byref(c), fp(query), fp(out),
                                                  C.byref(err), None))
            self.last_max_error = err.value
        return out

    def close(self):
        if self.h:
            self.o.fn("paged_destroy", None)(self.h)
            self.h = None


class Ref(_Base):
    """The unmodified reference behind oracle/ref_harness.cpp."""
    prefix = "sfref_"
    kind = "reference"

    @staticmethod
    def available():
        return os.path.exists(REF_SO)

    def __init__(self):
        super().__init__(REF_SO)

    def _check(self, status):
        if status != 0:
            raise OracleError(status, self.fn("last_error", C.c_char_p)().decode())

    def round_bf16(self, a):
        a = f32(a).copy()
        self.fn("round_bf16", None)(fp(a), C.c_longlong(a.size))
        return a

    def make_decoder_data(self, c, seed):
        shapes = decoder_shapes(c)
        data = {n: np.zeros(shapes[n], np.float32) for n in shapes}
        args = [fp(data.get(n)) for n in DATA_FIELDS]
        self._check(self.fn("make_decoder_data")(C.byref(c), C.c_uint(seed), *args))
        return data

    def make_attention_data(self, c, seed):
        q = np.empty((c.batch, c.query_heads, c.sequence_query, c.head_dim), np.float32)
        k = np.empty((c.batch, c.kv_heads, c.sequence_kv, c.head_dim), np.float32)
        v = np.empty((c.batch, c.kv_heads, c.sequence_kv, c.head_dim_value), np.float32)
        self._check(self.fn("make_attention_data")(C.byref(c), C.c_uint(seed), fp(q), fp(k), fp(v)))
        return q, k, v

    def make_moe_data(self, c, seed):
        h, i, e = c.hidden, c.intermediate, c.experts
        d = {"input": np.empty((c.tokens, h), np.float32), "router_weight": np.empty((h, e), np.float32),
             "w1": np.empty((e, h, i), np.float32), "w3": np.empty((e, h, i), np.float32),
             "w2": np.empty((e, i, h), np.float32)}
        self._check(self.fn("make_moe_data")(C.byref(c), C.c_uint(seed), fp(d["input"]),
                                             fp(d["router_weight"]), fp(d["w1"]), fp(d["w3"]), fp(d["w2"])))
        return d

    def import_stablehlo(self, text, moe=False):
        flags, counts = np.zeros(3, np.int32), np.zeros(4, np.int32)
        self._check(self.fn("import_stablehlo")(text.encode(), int(moe), ip(flags), ip(counts)))
        return {"fused_qkv": bool(flags[0]), "fused_gate_up": bool(flags[1]),
                "fused_rope": bool(flags[2]), "operations": int(counts[0]), "values": int(counts[1]),
                "inputs": int(counts[2]), "matmuls": int(counts[3])}

    def canonical_graph_names(self, c):
        buf = C.create_string_buffer(8192)
        self._check(self.fn("canonical_graph_names")(C.byref(c), buf, 8192))
        return buf.value.decode().split()

    def rms_norm(self, x, w, eps):
        x, w = f32(x), f32(w)
        out = np.empty_like(x)
        self._check(self.fn("rms_norm")(fp(x), fp(w), x.shape[0], x.shape[1], C.c_float(eps), fp(out)))
        return out

    def matmul(self, a, b, fma=False, threads=0):
        a, b = f32(a), f32(b)
        c = np.empty((a.shape[0], b.shape[1]), np.float32)
        if fma:
            self._check(self.fn("gemm_native")(a.shape[0], b.shape[1], a.shape[1], fp(a), fp(b), fp(c), threads))
        else:
            self._check(self.fn("scalar_matmul")(a.shape[0], b.shape[1], a.shape[1], fp(a), fp(b), fp(c)))
        return c

    def split_qkv_rope(self, c, fused):
        fused = f32(fused)
        q = np.empty((c.batch, c.query_heads, c.sequence, c.head_dim), np.float32)
        k = np.empty((c.batch, c.kv_heads, c.sequence, c.head_dim), np.float32)
        v = np.empty_like(k)
        self._check(self.fn("split_qkv_rope")(C.byref(c), fp(fused), fp(q), fp(k), fp(v)))
        return q, k, v

    def swiglu(self, gate_up, intermediate):
        gate_up = f32(gate_up)
        out = np.empty((gate_up.shape[0], intermediate), np.float32)
        self._check(self.fn("swiglu")(fp(gate_up), gate_up.shape[0], intermediate, fp(out)))
        return out

    def attention_reference(self, c, q, k, v, threads=0):
        q, k, v = f32(q), f32(k), f32(v)
        out = np.empty((c.batch, c.query_heads, c.sequence_query, c.head_dim_value), np.float32)
        self._check(self.fn("reference_attention")(C.byref(c), fp(q), fp(k), fp(v), fp(out)))
        return out

    def execute_attention(self, c, q, k, v, strategy=-1, query_tile=0, kv_tile=0, threads=0):
        """Returns (output, milliseconds, strategy used)."""
        q, k, v = f32(q), f32(k), f32(v)
        out = np.empty((c.batch, c.query_heads, c.sequence_query, c.head_dim_value), np.float32)
        ms, used = C.c_double(0), C.c_int(0)
        self._check(self.fn("execute_attention")(C.byref(c), strategy, query_tile, kv_tile, threads,
                                                 fp(q), fp(k), fp(v), fp(out), C.byref(ms), C.byref(used)))
        return out, ms.value, used.value

    def attention_materialized(self, c, q, k, v):
        return self.execute_attention(c, q, k, v, strategy=0)[0]

    def attention_io_aware(self, c, q, k, v, query_tile, kv_tile, threads=0):
        return self.execute_attention(c, q, k, v, 2, query_tile, kv_tile, threads)[0]

    def decode_attention(self, c, q, keys, values, length, capacity=0, threads=0):
        q, keys, values = f32(q), f32(keys), f32(values)
        out = np.empty((c.batch, c.query_heads, c.sequence_query, c.head_dim_value), np.float32)
        split = C.c_int(0)
        self._check(self.fn("decode_attention")(C.byref(c), capacity, fp(q), fp(keys), fp(values),
                                                length, threads, fp(out), C.byref(split)))
        return out

    def paged_create(self, batch, kv_heads, dim, dim_v, page_tokens, capacity):
        h = self.fn("paged_create", C.c_void_p)(batch, kv_heads, dim, dim_v, page_tokens, capacity)
        if not h:
            raise OracleError(1, self.fn("last_error", C.c_char_p)().decode())
        return PagedHandle(self, h, (batch, kv_heads, dim, dim_v, page_tokens, capacity))

    def route_topk(self, c, x, router_weight, bias=None):
        assert bias is None, "the reference has no router bias"
        x, router_weight = f32(x), f32(router_weight)
        tokens = x.shape[0]
        ids = np.empty((tokens, c.top_k), np.int32)
        weights = np.empty((tokens, c.top_k), np.float32)
        counts = np.empty(c.experts, np.int32)
        self._check(self.fn("route_topk")(C.byref(c), fp(x), tokens, fp(router_weight), ip(ids),
                                          fp(weights), ip(counts)))
        return ids, weights, counts

    def make_routing_trace(self, c, distribution, seed):
        ids = np.empty((c.tokens, c.top_k), np.int32)
        weights = np.empty((c.tokens, c.top_k), np.float32)
        counts = np.empty(c.experts, np.int32)
        self._check(self.fn("make_routing_trace")(C.byref(c), distribution, C.c_uint(seed), ip(ids),
                                                  fp(weights), ip(counts)))
        return ids, weights, counts

    def decoder_profiles(self):
        """realistic_decoder_profiles as text lines, then the headers of the two CSV writers and the
        compile-only row of profile 14 (see sfref_decoder_profiles)."""
        buf = C.create_string_buffer(1 << 16)
        self._check(self.fn("decoder_profiles")(buf, len(buf)))
        return buf.value.decode()

    def dispatch_tokens(self, c, x, ids, weights, counts, copy_values=True):
        x, ids, weights, counts = f32(x), i32(ids), f32(weights), i32(counts)
        tokens = ids.shape[0]
        n = tokens * c.top_k
        values = np.empty((n, c.hidden), np.float32)
        offsets = np.empty(c.experts + 1, np.int32)
        token_ids, slots = np.empty(n, np.int32), np.empty(n, np.int32)
        rw = np.empty(n, np.float32)
        self._check(self.fn("dispatch_tokens")(C.byref(c), fp(x), tokens, ip(ids), fp(weights),
                                               ip(counts), fp(values), ip(offsets), ip(token_ids),
                                               ip(slots), fp(rw)))
        return values, offsets, token_ids, slots, rw

    def plan_moe_tasks(self, c, ids, weights, counts, split_threshold=0):
        ids, weights, counts = i32(ids), f32(weights), i32(counts)
        tasks = np.empty((4096, 4), np.int32)
        n = C.c_int(0)
        self._check(self.fn("plan_moe_tasks")(C.byref(c), ids.shape[0], ip(ids), fp(weights),
                                              ip(counts), split_threshold, ip(tasks), 4096, C.byref(n)))
        return tasks[:n.value].copy()

    def moe_reference(self, c, x, w1, w3, w2, ids, weights, counts=None, threads=0):
        x, w1, w3, w2, ids, weights = f32(x), f32(w1), f32(w3), f32(w2), i32(ids), f32(weights)
        counts = i32(counts) if counts is not None else np.bincount(ids.ravel(), minlength=c.experts).astype(np.int32)
        router = np.zeros((c.hidden, c.experts), np.float32)
        out = np.empty((x.shape[0], c.hidden), np.float32)
        self._check(self.fn("reference_moe")(C.byref(c), fp(x), x.shape[0], fp(router), fp(w1), fp(w3),
                                             fp(w2), ip(ids), fp(weights), ip(counts), fp(out)))
        return out

    def moe_grouped(self, c, x, w1, w3, w2, ids, weights, counts, threads=0, want_ms=False):
        x, w1, w3, w2 = f32(x), f32(w1), f32(w3), f32(w2)
        ids, weights, counts = i32(ids), f32(weights), i32(counts)
        router = np.zeros((c.hidden, c.experts), np.float32)
        out = np.empty((x.shape[0], c.hidden), np.float32)
        ms = (C.c_double * 4)()
        self._check(self.fn("execute_moe")(C.byref(c), fp(x), x.shape[0], fp(router), fp(w1), fp(w3),
                                           fp(w2), ip(ids), fp(weights), ip(counts), threads, fp(out), ms))
        return (out, list(ms)) if want_ms else out

    def moe_quantized(self, c, x, w1, w3, w2, ids, weights, counts=None, per_channel=True):
        """quantize_moe_weights + execute_quantized_moe (src/next_milestones.cpp:699-738);
        returns (output, max error against reference_moe on the unquantized weights)."""
        x, w1, w3, w2, ids, weights = f32(x), f32(w1), f32(w3), f32(w2), i32(ids), f32(weights)
        counts = i32(counts) if counts is not None else np.bincount(ids.ravel(), minlength=c.experts).astype(np.int32)
        out = np.empty((x.shape[0], c.hidden), np.float32)
        err = C.c_double(0)
        self._check(self.fn("quantized_moe")(C.byref(c), fp(x), x.shape[0], fp(w1), fp(w3), fp(w2), ip(ids),
                                             fp(weights), ip(counts), int(per_channel), fp(out), C.byref(err)))
        return out, err.value

    def decoder_create(self, c, data, stablehlo_text="", threads=0, trace=None):
        d, keep = pack_decoder_data(data, trace)
        h = self.fn("decoder_create", C.c_void_p)(C.byref(c), C.byref(d), stablehlo_text.encode(), threads)
        del keep
        if not h:
            raise OracleError(1, self.fn("last_error", C.c_char_p)().decode())
        return RefDecoder(self, h, c)

    def decoder_layer(self, c, data, native=False, threads=0, trace=None, stablehlo_text=""):
        dec = self.decoder_create(c, data, stablehlo_text, threads, trace)
        try:
            return dec.execute_once()[0] if native else dec.reference()
        finally:
            dec.close()


class RefDecoder:
    def __init__(self, owner, handle, c):
        self.o, self.h, self.c = owner, C.c_void_p(handle), c

    def execute_once(self):
        out = np.empty((self.c.batch * self.c.sequence, self.c.hidden), np.float32)
        ms = (C.c_double * 6)()
        self.o._check(self.o.fn("decoder_execute_once")(self.h, fp(out), ms))
        return out, list(ms)

    def reference(self):
        out = np.empty((self.c.batch * self.c.sequence, self.c.hidden), np.float32)
        self.o._check(self.o.fn("decoder_reference")(self.h, fp(out)))
        return out

    def quantized(self, per_channel=True):
        """Weight-only INT8 layer of the reference; returns (output, max error vs its scalar reference)."""
        out = np.empty((self.c.batch * self.c.sequence, self.c.hidden), np.float32)
        err = C.c_double(0)
        self.o._check(self.o.fn("decoder_quantized")(self.h, int(per_channel), fp(out), C.byref(err)))
        return out, err.value

    def plan_info(self):
        s, k, w = C.c_int(0), C.c_int(0), C.c_longlong(0)
        self.o._check(self.o.fn("decoder_plan_info")(self.h, C.byref(s), C.byref(k), C.byref(w)))
        return {"attention_strategy": s.value, "split_kv": k.value, "workspace_bytes": w.value}

    def close(self):
        if self.h:
            self.o.fn("decoder_destroy", None)(self.h)
            self.h = None
