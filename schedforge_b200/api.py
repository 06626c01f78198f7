"""Python face of the C ABI, named after the reference's C++ entry points
(StableHLOImporter, DecoderCompiler.compile, execute_decoder_layer, execute_attention,
PagedKVCache, route_topk, dispatch_tokens, execute_moe).  Everything here is a thin
ctypes call into libschedforge_b200.so; there is no Python or CPU compute path."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as L


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _fp(a):
    return None if a is None else a.ctypes.data_as(L.f32p)


def _ip(a):
    return None if a is None else a.ctypes.data_as(L.i32p)


def decoder_config(batch=1, sequence=16, hidden=64, intermediate=128, query_heads=4, kv_heads=2,
                   head_dim=16, rms_epsilon=1e-5, rope_theta=10000.0, causal=True, moe=False, experts=4,
                   top_k=2, context_sequence=0):
    """DecoderConfig (include/schedforge/decoder_compiler.h:17-32 of the reference)."""
    return L.DecoderConfig(batch, sequence, hidden, intermediate, query_heads, kv_heads, head_dim,
                           rms_epsilon, rope_theta, int(causal), int(moe), experts, top_k, context_sequence)


def compile_options(dtype=L.BF16, token_major_attention=True, fuse_epilogues=True, gemm_backend=L.GEMM_AUTO,
                    attention_backend=0, page_tokens=16, tp_rank=0, tp_size=1, seed_block_table=0,
                    no_workspace_reuse=False, no_pipeline=False, append_new_token=False, weight_int8=False,
                    kv_capacity=0, norm_fusion=None, local_expert_weights=False, fixed_order=False):
    return L.CompileOptions(dtype, int(token_major_attention), int(fuse_epilogues), gemm_backend,
                            attention_backend, page_tokens, tp_rank, tp_size, seed_block_table,
                            int(no_workspace_reuse), int(no_pipeline), int(append_new_token), int(weight_int8),
                            int(kv_capacity), 0 if norm_fusion is None else (1 if norm_fusion else -1), int(local_expert_weights),
                            int(fixed_order))


class StableHLOImporter:
    """StableHLOImporter::importText + DecoderFusionPass::run."""

    @staticmethod
    def import_text(text):
        s = L.GraphSummary()
        L.check(L.load().sfb_import_stablehlo(text.encode(), C.byref(s)))
        return {n: (bool(getattr(s, n)) if n.startswith("fused") else getattr(s, n)) for n, _ in s._fields_}

    @staticmethod
    def dump(text):
        buf = C.create_string_buffer(1 << 16)
        L.check(L.load().sfb_import_stablehlo_dump(text.encode(), buf, C.c_size_t(len(buf))))
        return buf.value.decode()


class DecoderExecutablePlan:
    """Owns an sfb_decoder_plan.  Build with DecoderCompiler.compile."""

    def __init__(self, handle, config, options, keep):
        self._h = handle
        self.config = config
        self.options = options
        self._keep = keep
        self._callback = None

    @property
    def rows(self):
        return self.config.batch * self.config.sequence

    def execute(self, x, out=None, trace=None):
        """execute_decoder_layer, one repetition: host input [T,H] -> (host output, DecoderResult)."""
        x = _f32(x) if not isinstance(x, np.ndarray) or x.dtype != np.float32 or not x.flags.c_contiguous else x
        if out is None:
            out = np.empty((self.rows, self.config.hidden), np.float32)
        result = L.DecoderResult()
        ids = weights = counts = None
        if trace is not None:
            ids, weights, counts = _i32(trace[0]), _f32(trace[1]), _i32(trace[2])
        L.check(L.load().sfb_decoder_execute(self._h, _fp(x), _fp(out), _ip(ids), _fp(weights), _ip(counts),
                                             C.byref(result)))
        return out, result

    def step(self, x, out=None):
        """One autoregressive step (sfb_decoder_step): appends the token's K/V, attends, advances the cache."""
        x = _f32(x)
        if out is None:
            out = np.empty((self.rows, self.config.hidden), np.float32)
        result = L.DecoderResult()
        L.check(L.load().sfb_decoder_step(self._h, _fp(x), _fp(out), C.byref(result)))
        return out, result

    def kv_info(self):
        info = np.zeros(4, np.int32)
        table, free = np.zeros(65536, np.int32), np.zeros(65536, np.int32)
        L.check(L.load().sfb_decoder_kv_info(self._h, _ip(info), _ip(table), table.size, _ip(free), free.size))
        return {"length": int(info[0]), "page_table": table[:info[1]].copy(), "free_pages": free[:info[2]].copy(),
                "pages": int(info[3])}

    def kv_truncate(self, new_length):
        L.check(L.load().sfb_decoder_kv_truncate(self._h, int(new_length)))

    def kv_release(self, pages):
        pages = _i32(pages)
        L.check(L.load().sfb_decoder_kv_release(self._h, _ip(pages), pages.size))

    def execute_ptr(self, in_ptr, out_ptr, result=None):
        """Same call with raw host addresses (e.g. pinned torch tensors)."""
        L.check(L.load().sfb_decoder_execute(self._h, C.c_void_p(in_ptr), C.c_void_p(out_ptr), None, None, None,
                                             C.byref(result) if result is not None else None))

    def execute_rows_ptr(self, in_ptr, out_ptr, row_begin, row_count, result=None):
        """This rank's rows of the input in, the same rows of the output out (raw host addresses); see
        sfb_decoder_execute_rows."""
        L.check(L.load().sfb_decoder_execute_rows(self._h, C.c_void_p(in_ptr), C.c_void_p(out_ptr), row_begin, row_count,
                                                  C.byref(result) if result is not None else None))

    def execute_rows(self, x_rows, row_begin):
        x_rows = _f32(x_rows)
        out = np.empty_like(x_rows)
        result = L.DecoderResult()
        self.execute_rows_ptr(x_rows.ctypes.data, out.ctypes.data, row_begin, x_rows.shape[0], result)
        return out, result

    def upload_input(self, x):
        x = _f32(x)
        L.check(L.load().sfb_decoder_upload_input(self._h, _fp(x)))

    def execute_resident(self, stream=None):
        L.check(L.load().sfb_decoder_execute_resident(self._h, C.c_void_p(stream)))

    def download_output(self):
        out = np.empty((self.rows, self.config.hidden), np.float32)
        L.check(L.load().sfb_decoder_download_output(self._h, _fp(out)))
        return out

    def set_allreduce(self, fn):
        """fn(buffer_ptr, count, dtype, stream_ptr) must all-reduce (sum) in place on that stream."""
        if fn is None:
            self._callback = None
            L.check(L.load().sfb_decoder_set_allreduce(self._h, None, None))
            return
        self._callback = L.ALLREDUCE_FN(lambda user, buf, count, dtype, stream: fn(buf, count, dtype, stream))
        L.check(L.load().sfb_decoder_set_allreduce(self._h, self._callback, None))

    def enable_peer_allreduce(self, rank, world, exchange, mode=1):
        """Fused all-reduce over NVLink peer memory for the O and Down projections of a sharded plan.
        mode 1 = one-shot, 2 = two-shot (reduce-scatter under the GEMM, sum + all-gather by the row owners),
        0 = pick (sfb_decoder_set_peer_collective).

        exchange(handle: bytes) -> list of every rank's 64-byte handle in rank order (for instance
        torch.distributed.all_gather_object).  Every rank must call this at the same point."""
        lib = L.load()
        nbytes = lib.sfb_decoder_peer_bytes(self._h)
        local, handle = C.c_void_p(), C.create_string_buffer(64)
        L.check(lib.sfb_peer_alloc(C.c_size_t(nbytes), C.byref(local), handle))
        handles = exchange(handle.raw)
        bases = (C.c_void_p * world)()
        self._peer_mapped = []
        for s in range(world):
            if s == rank:
                continue
            mapped = C.c_void_p()
            L.check(lib.sfb_peer_open(C.create_string_buffer(handles[s], 64), C.byref(mapped)))
            bases[s] = mapped.value
            self._peer_mapped.append(mapped)
        self._peer_local = local
        L.check(lib.sfb_decoder_set_peer_collective(self._h, local, bases, int(mode)))

    def disable_peer_allreduce(self):
        """Unmaps the peers' buffers and frees the local one (call on every rank after a barrier)."""
        lib = L.load()
        if getattr(self, "_peer_local", None) is None:
            return
        L.check(lib.sfb_decoder_set_peer_allreduce(self._h, None, None))
        for mapped in self._peer_mapped:
            L.check(lib.sfb_peer_close(mapped))
        L.check(lib.sfb_peer_free(self._peer_local))
        self._peer_local, self._peer_mapped = None, []

    def read_tensor(self, name, dtype=np.float32):
        count = C.c_int64(0)
        L.check(L.load().sfb_decoder_read_tensor(self._h, name.encode(), None, C.c_int64(0), C.byref(count)))
        out = np.empty(count.value, np.float32)
        L.check(L.load().sfb_decoder_read_tensor(self._h, name.encode(), _fp(out), C.c_int64(out.size), C.byref(count)))
        return out.view(np.int32) if dtype == np.int32 else out

    def dump(self):
        buf = C.create_string_buffer(1 << 17)
        L.check(L.load().sfb_decoder_dump(self._h, buf, C.c_size_t(len(buf))))
        return buf.value.decode()

    @property
    def workspace_bytes(self):
        return L.load().sfb_decoder_workspace_bytes(self._h)

    @property
    def stream(self):
        return L.load().sfb_decoder_stream(self._h)

    def close(self):
        if self._h:
            L.load().sfb_decoder_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DecoderCompiler:
    """DecoderCompiler::compile: `data` maps DecoderData field names to float32 arrays."""

    @staticmethod
    def compile(config, data, stablehlo_text="", options=None):
        options = options or compile_options()
        keep = {k: _f32(v) for k, v in data.items() if v is not None and k in L.DATA_FIELDS}
        d = L.DecoderData()
        for name in L.DATA_FIELDS:
            setattr(d, name, _fp(keep.get(name)))
        handle = C.c_void_p()
        L.check(L.load().sfb_decoder_compile(C.byref(config), C.byref(d), stablehlo_text.encode(),
                                             C.byref(options), C.byref(handle)))
        return DecoderExecutablePlan(handle, config, options, None)


class ExecutablePlanOptimizer:
    """ExecutablePlanOptimizer::optimize: returns (winning plan, OptimizationResult, candidates)."""

    @staticmethod
    def optimize(config, data, x, stablehlo_text="", options=None, measurement_budget=8, repetitions=2):
        options = options or compile_options()
        keep = {k: _f32(v) for k, v in data.items() if v is not None and k in L.DATA_FIELDS}
        d = L.DecoderData()
        for name in L.DATA_FIELDS:
            setattr(d, name, _fp(keep.get(name)))
        x = _f32(x)
        result = L.OptimizationResult()
        candidates = (L.PlanCandidate * 17)()
        handle = C.c_void_p()
        L.check(L.load().sfb_decoder_optimize(C.byref(config), C.byref(d), stablehlo_text.encode(), C.byref(options),
                                              _fp(x), measurement_budget, repetitions, C.byref(result), candidates, 17,
                                              C.byref(handle)))
        return DecoderExecutablePlan(handle, config, result.winner_options, None), result, list(candidates)[:result.candidates]


def execute_decoder_layer(plan, x, trace=None):
    return plan.execute(x, trace=trace)


def attention_config(batch, query_heads, kv_heads, sequence_query, sequence_kv, head_dim, head_dim_value=None,
                     causal=False, scale=0.0):
    return L.AttentionConfig(batch, query_heads, kv_heads, sequence_query, sequence_kv, head_dim,
                             head_dim_value or head_dim, int(causal), scale)


def execute_attention(config, q, k, v, dtype=L.F32, backend=0):
    """execute_attention: q [B,Hq,Sq,D], k [B,Hkv,Sk,D], v [B,Hkv,Sk,Dv] -> (out [B,Hq,Sq,Dv], ms)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty((config.batch, config.query_heads, config.sequence_query, config.head_dim_value), np.float32)
    ms = C.c_double(0)
    L.check(L.load().sfb_attention_execute(C.byref(config), _fp(q), _fp(k), _fp(v), _fp(out), dtype, backend,
                                           C.byref(ms)))
    return out, ms.value


def execute_decode_attention(config, q, keys, values, length, dtype=L.F32):
    q, keys, values = _f32(q), _f32(keys), _f32(values)
    out = np.empty((config.batch, config.query_heads, config.sequence_query, config.head_dim_value), np.float32)
    ms = C.c_double(0)
    L.check(L.load().sfb_attention_decode(C.byref(config), _fp(q), _fp(keys), _fp(values), length, _fp(out), dtype,
                                          C.byref(ms)))
    return out, ms.value


class PagedKVCache:
    """PagedKVCache + append_paged_kv / truncate / release / gather / execute_paged_decode_attention."""

    def __init__(self, batch, kv_heads, head_dim, head_dim_value, page_tokens, capacity, dtype=L.F32):
        self.shape = (batch, kv_heads, head_dim, head_dim_value, page_tokens, capacity)
        self._h = C.c_void_p()
        L.check(L.load().sfb_paged_create(batch, kv_heads, head_dim, head_dim_value, page_tokens, capacity, dtype,
                                          C.byref(self._h)))

    def set_free_pages(self, pages):
        pages = _i32(pages)
        L.check(L.load().sfb_paged_set_free_pages(self._h, _ip(pages), pages.size))

    def append(self, keys, values, tokens):
        keys, values = _f32(keys), _f32(values)
        L.check(L.load().sfb_paged_append(self._h, _fp(keys), _fp(values), tokens))

    def truncate(self, new_length):
        L.check(L.load().sfb_paged_truncate(self._h, new_length))

    def release(self, pages):
        pages = _i32(pages)
        L.check(L.load().sfb_paged_release(self._h, _ip(pages), pages.size))

    def info(self):
        info = np.zeros(4, np.int32)
        table, free = np.zeros(65536, np.int32), np.zeros(65536, np.int32)
        L.check(L.load().sfb_paged_info(self._h, _ip(info), _ip(table), table.size, _ip(free), free.size))
        return {"length": int(info[0]), "page_table": table[:info[1]].copy(), "free_pages": free[:info[2]].copy(),
                "pages": int(info[3])}

    def gather(self):
        b, hkv, d, dv, _, _ = self.shape
        n = self.info()["length"]
        keys, values = np.empty((b, hkv, max(n, 1), d), np.float32), np.empty((b, hkv, max(n, 1), dv), np.float32)
        L.check(L.load().sfb_paged_gather(self._h, _fp(keys), _fp(values)))
        return keys, values

    def decode(self, config, q):
        q = _f32(q)
        out = np.empty((config.batch, config.query_heads, config.sequence_query, config.head_dim_value), np.float32)
        ms = C.c_double(0)
        L.check(L.load().sfb_paged_decode(self._h, C.byref(config), _fp(q), _fp(out), C.byref(ms)))
        return out, ms.value

    def close(self):
        if self._h:
            L.load().sfb_paged_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def moe_config(tokens, hidden, intermediate, experts, top_k):
    return L.MoeConfig(tokens, hidden, intermediate, experts, top_k)


def route_topk(config, x, router_weight, router_bias=None, dtype=L.F32):
    x, router_weight = _f32(x), _f32(router_weight)
    bias = _f32(router_bias) if router_bias is not None else None
    tokens = x.shape[0]
    ids, weights = np.empty((tokens, config.top_k), np.int32), np.empty((tokens, config.top_k), np.float32)
    counts = np.empty(config.experts, np.int32)
    L.check(L.load().sfb_moe_route_topk(C.byref(config), _fp(x), tokens, _fp(router_weight), _fp(bias), dtype,
                                        _ip(ids), _fp(weights), _ip(counts)))
    return ids, weights, counts


def dispatch_tokens(config, x, ids, weights, counts, dtype=L.F32, copy_values=True):
    ids, weights, counts = _i32(ids), _f32(weights), _i32(counts)
    tokens = ids.shape[0]
    n = tokens * config.top_k
    x = _f32(x) if x is not None else None
    values = np.empty((n, config.hidden), np.float32) if copy_values else None
    offsets = np.empty(config.experts + 1, np.int32)
    token_ids, slots, rw = np.empty(n, np.int32), np.empty(n, np.int32), np.empty(n, np.float32)
    L.check(L.load().sfb_moe_dispatch_tokens(C.byref(config), _fp(x), tokens, _ip(ids), _fp(weights), _ip(counts),
                                             dtype, _fp(values), _ip(offsets), _ip(token_ids), _ip(slots), _fp(rw)))
    return values, offsets, token_ids, slots, rw


def execute_moe(config, x, w1, w3, w2, ids, weights, counts, dtype=L.F32, gemm_backend=L.GEMM_AUTO):
    x, w1, w3, w2 = _f32(x), _f32(w1), _f32(w3), _f32(w2)
    ids, weights, counts = _i32(ids), _f32(weights), _i32(counts)
    out = np.empty((x.shape[0], config.hidden), np.float32)
    ms = C.c_double(0)
    L.check(L.load().sfb_moe_execute(C.byref(config), _fp(x), x.shape[0], _fp(w1), _fp(w3), _fp(w2), _ip(ids),
                                     _fp(weights), _ip(counts), dtype, gemm_backend, _fp(out), C.byref(ms)))
    return out, ms.value


class MoeExecutablePlan:
    """MoeCompiler.compile + execute_moe on a plan that keeps the packed expert weights on the device."""

    def __init__(self, config, w1, w3, w2, router_weight=None, router_bias=None, dtype=L.BF16, gemm_backend=L.GEMM_AUTO,
                 weight_int8=False):
        self.config = config
        self._h = C.c_void_p()
        w1, w3, w2 = _f32(w1), _f32(w3), _f32(w2)
        rw = _f32(router_weight) if router_weight is not None else None
        rb = _f32(router_bias) if router_bias is not None else None
        L.check(L.load().sfb_moe_compile(C.byref(config), _fp(w1), _fp(w3), _fp(w2), _fp(rw), _fp(rb), dtype, gemm_backend,
                                         int(weight_int8), C.byref(self._h)))

    def execute(self, x, trace=None):
        """One pass: with trace = (ids, weights, counts) the router is skipped, else the plan routes itself."""
        x = _f32(x)
        out = np.empty((x.shape[0], self.config.hidden), np.float32)
        ms = C.c_double(0)
        ids = weights = counts = None
        if trace is not None:
            ids, weights, counts = _i32(trace[0]), _f32(trace[1]), _i32(trace[2])
        L.check(L.load().sfb_moe_plan_execute(self._h, _fp(x), x.shape[0], _ip(ids), _fp(weights), _ip(counts), _fp(out),
                                              C.byref(ms)))
        return out, ms.value

    def close(self):
        if self._h:
            L.load().sfb_moe_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def execute_quantized_moe(config, x, w1, w3, w2, ids, weights, counts, per_channel=True, gemm_backend=L.GEMM_AUTO):
    """quantize_moe_weights + execute_quantized_moe of the reference (src/next_milestones.cpp:699-738):
    the experts multiply by the INT8 round trip of their weights."""
    x, w1, w3, w2 = _f32(x), _f32(w1), _f32(w3), _f32(w2)
    ids, weights, counts = _i32(ids), _f32(weights), _i32(counts)
    out = np.empty((x.shape[0], config.hidden), np.float32)
    ms = C.c_double(0)
    L.check(L.load().sfb_moe_execute_quantized(C.byref(config), _fp(x), x.shape[0], _fp(w1), _fp(w3), _fp(w2),
                                               _ip(ids), _fp(weights), _ip(counts), int(per_channel), gemm_backend,
                                               _fp(out), C.byref(ms)))
    return out, ms.value


def plan_moe_tasks(config, counts, split_threshold=0):
    counts = _i32(counts)
    tasks = np.empty((4096, 4), np.int32)
    n = C.c_int(0)
    L.check(L.load().sfb_moe_plan_tasks(C.byref(config), _ip(counts), split_threshold, _ip(tasks), 4096, C.byref(n)))
    return tasks[:n.value].copy()


def make_routing_trace(config, distribution, seed):
    """make_routing_trace of the reference (distribution 0 uniform, 1 moderate-skew, 2 heavy-skew)."""
    ids = np.empty((config.tokens, config.top_k), np.int32)
    weights = np.empty((config.tokens, config.top_k), np.float32)
    counts = np.empty(config.experts, np.int32)
    L.check(L.load().sfb_make_routing_trace(C.byref(config), distribution, C.c_uint(seed), _ip(ids), _fp(weights),
                                            _ip(counts)))
    return ids, weights, counts


def make_decoder_input(config, seed):
    """The input tensor make_decoder_data of the reference draws for this configuration and seed."""
    x = np.empty((config.batch * config.sequence, config.hidden), np.float32)
    L.check(L.load().sfb_make_decoder_input(C.byref(config), C.c_uint(seed), _fp(x)))
    return x


def make_decoder_data(config, seed):
    """make_decoder_data of the reference (same seeded streams): dict of float32 arrays incl. "input"."""
    t, h, i = config.batch * config.sequence, config.hidden, config.intermediate
    kv = config.kv_heads * config.head_dim
    sizes = {"input": t * h, "rms1_weight": h, "rms2_weight": h, "query_weight": h * h, "key_weight": h * kv,
             "value_weight": h * kv, "output_weight": h * h, "gate_weight": h * i, "up_weight": h * i, "down_weight": i * h}
    if config.ffn_moe:
        e = config.experts
        sizes.update(router_weight=h * e, w1=e * h * i, w3=e * h * i, w2=e * i * h)
    if config.context_sequence > 0:
        n = config.batch * config.kv_heads * config.context_sequence * config.head_dim
        sizes.update(cached_key=n, cached_value=n)
    data = {k: np.zeros(n, np.float32) for k, n in sizes.items()}
    buffers = L.DecoderDataBuffers()
    for name in L.DATA_BUFFER_FIELDS:
        if name in data:
            setattr(buffers, name, _fp(data[name]))
    L.check(L.load().sfb_make_decoder_data(C.byref(config), C.c_uint(seed), _fp(data["input"]), C.byref(buffers)))
    return data


def realistic_decoder_profiles():
    """realistic_decoder_profiles of the reference: 24 DecoderProfile records."""
    lib = L.load()
    out = []
    for index in range(lib.sfb_decoder_profile_count()):
        p = L.DecoderProfile()
        L.check(lib.sfb_decoder_profile_get(index, C.byref(p)))
        out.append(p)
    return out


def benchmark_decoder_profile(profile, stablehlo_text="", options=None, max_real_flops=1 << 62,
                              max_real_weight_bytes=1 << 62, optimize_plan=False, repetitions=3):
    """benchmark_decoder_profile of the reference on the device plan; returns a DecoderBenchmarkRecord."""
    record = L.DecoderBenchmarkRecord()
    L.check(L.load().sfb_benchmark_decoder_profile(C.byref(profile), stablehlo_text.encode() or None,
                                                   C.byref(options) if options is not None else None,
                                                   max_real_flops, max_real_weight_bytes, int(optimize_plan),
                                                   repetitions, C.byref(record)))
    return record


def _record_array(records):
    array = (L.DecoderBenchmarkRecord * max(1, len(records)))()
    for i, r in enumerate(records):
        C.memmove(C.byref(array[i]), C.byref(r), C.sizeof(L.DecoderBenchmarkRecord))
    return array


def write_decoder_benchmark_csv(path, records):
    L.check(L.load().sfb_write_decoder_benchmark_csv(str(path).encode(), _record_array(records), len(records)))


def write_decoder_plan_candidates_csv(path, records):
    L.check(L.load().sfb_write_decoder_plan_candidates_csv(str(path).encode(), _record_array(records), len(records)))


def shard_columns(a, rank, size):
    a = _f32(a)
    out = np.empty((a.shape[0], a.shape[1] // size), np.float32)
    L.check(L.load().sfb_shard_columns(_fp(a), a.shape[0], a.shape[1], rank, size, _fp(out)))
    return out


def shard_rows(a, rank, size):
    a = _f32(a)
    out = np.empty((a.shape[0] // size, a.shape[1]), np.float32)
    L.check(L.load().sfb_shard_rows(_fp(a), a.shape[0], a.shape[1], rank, size, _fp(out)))
    return out
