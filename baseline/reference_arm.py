"""The reference arm of bench.py: the reference's own CUDA backend (built unmodified by
baseline/build_reference.py) driven through its C ABI, backend/shim.h: te_init,
te_model_create, te_model_load_tensor, te_model_finalize, te_forward_batch.  That ABI is
what the reference's Go engine calls (engine/engine.go steps a batch with one
te_forward_batch); block tables and positions are the caller's, here as there.  The
reference computes in float32 (cuBLAS SGEMM and its own SIMT kernels) and returns the
logits of every sequence's last token to the host each step; both belong to its stock
path and stay inside the timed region.  te_forward_batch is synchronous, so steps are
timed by the wall clock around the call.
"""
from __future__ import annotations

import ctypes
import os
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_ref", "libkllm_backend.so")


class TeModelConfig(ctypes.Structure):        # field order of backend/shim.h:42-69
    _fields_ = [(n, ctypes.c_int64) for n in (
        "hidden", "n_layers", "n_heads", "n_kv_heads", "head_dim", "intermediate", "vocab", "max_seq",
        "n_experts", "top_k", "moe_intermediate", "router_mode", "kv_block_size", "kv_num_blocks", "arch",
        "sliding_window", "sliding_pattern")] + [(n, ctypes.c_double) for n in (
            "rope_theta", "rope_local_theta", "query_scalar", "rms_eps")]


def available() -> str:
    """'' when the arm can run, else why not (one line)."""
    if not os.path.isfile(LIB):
        return ("the reference is a Go program with a CUDA backend: pip reports 'not installable: neither setup.py "
                "nor pyproject.toml', no Go toolchain exists here, and baseline/_ref/libkllm_backend.so (its "
                "backend built by baseline/build_reference.py) is missing")
    return ""


class Reference:
    def __init__(self, cfg: dict, max_seqs: int, max_seq: int, block: int = 16, seed: int = 4, weights=None):
        """``weights``: tensor name -> float32 array to upload instead of random ones (a tied
        model's embedding goes in under ``lm_head.weight`` too, as tools/convert_hf.py:81-82
        resolves tying offline).  The backend holds one model per process."""
        self.lib = ctypes.CDLL(LIB)
        self.cfg, self.block, self.max_seq = cfg, block, max_seq
        self.blocks_per_seq = -(-max_seq // block)
        self._ok(self.lib.te_init(0))
        c = TeModelConfig()
        c.hidden, c.n_layers = cfg["hidden_size"], cfg["num_hidden_layers"]
        c.n_heads, c.n_kv_heads, c.head_dim = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        c.intermediate, c.vocab, c.max_seq = cfg["intermediate_size"], cfg["vocab_size"], max_seq
        c.kv_block_size, c.kv_num_blocks = block, max_seqs * self.blocks_per_seq
        c.rope_theta, c.rms_eps = float(cfg["rope_theta"]), float(cfg["rms_norm_eps"])
        self._ok(self.lib.te_model_create(ctypes.byref(c)))
        rng = np.random.default_rng(seed)
        d, f, v = c.hidden, c.intermediate, c.vocab
        qd, kd = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim

        def load(name, shape, gain=False):
            if weights is not None:
                src = "model.embed_tokens.weight" if name == "lm_head.weight" and name not in weights else name
                a = np.ascontiguousarray(weights[src], np.float32)
                assert a.shape == tuple(shape), f"{name}: {a.shape} is not {tuple(shape)}"
            else:
                a = np.ones(shape, np.float32) if gain else (rng.standard_normal(shape, dtype=np.float32) * 0.02)
            self._ok(self.lib.te_model_load_tensor(name.encode(), a.ctypes.data_as(ctypes.c_void_p),
                                                   ctypes.c_int64(a.size)))

        load("model.embed_tokens.weight", (v, d))
        for l in range(c.n_layers):
            p = f"model.layers.{l}."
            load(p + "input_layernorm.weight", (d,), gain=True)
            load(p + "post_attention_layernorm.weight", (d,), gain=True)
            for n, shape in (("q", (qd, d)), ("k", (kd, d)), ("v", (kd, d)), ("o", (d, qd))):
                load(p + f"self_attn.{n}_proj.weight", shape)
            for n, shape in (("gate", (f, d)), ("up", (f, d)), ("down", (d, f))):
                load(p + f"mlp.{n}_proj.weight", shape)
        load("model.norm.weight", (d,), gain=True)
        load("lm_head.weight", (v, d))
        self._ok(self.lib.te_model_finalize())
        self.vocab = v

    def _ok(self, rc):
        if rc != 0:
            buf = ctypes.create_string_buffer(512)
            self.lib.te_last_error(buf, 512)
            raise RuntimeError(f"reference backend: {buf.value.decode(errors='replace')} (code {rc})")

    def forward(self, tokens, n_tokens, pos, tables):
        """One te_forward_batch; returns the logits [n_seqs, vocab] it wrote to the host."""
        n_seqs = len(n_tokens)
        tok = np.ascontiguousarray(tokens, np.int32)
        nt = np.ascontiguousarray(n_tokens, np.int32)
        ps = np.ascontiguousarray(pos, np.int32)
        tb = np.ascontiguousarray(tables, np.int32)
        out = np.empty((n_seqs, self.vocab), np.float32)
        p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
        self._ok(self.lib.te_forward_batch(ctypes.c_int64(n_seqs), p(tok), p(nt), p(ps), p(tb),
                                           ctypes.c_int64(tb.shape[1]), p(out)))
        return out

    def debug(self, on: bool):
        """Switch the backend's debug taps (backend/shim.h:128-136)."""
        self._ok(self.lib.te_debug_set(ctypes.c_int64(1 if on else 0)))

    def taps(self):
        """What the last forward captured: the embedding output, the residual stream after
        every layer and the final norm's output, each [tokens of the step * hidden]."""
        self.lib.te_debug_count.restype = ctypes.c_int64
        self.lib.te_debug_size.restype = ctypes.c_int64
        out = []
        for i in range(int(self.lib.te_debug_count())):
            n = int(self.lib.te_debug_size(ctypes.c_int64(i)))
            a = np.empty(n, np.float32)
            self._ok(self.lib.te_debug_read(ctypes.c_int64(i), a.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(n)))
            out.append(a)
        return out

    def tables(self, n_seqs):
        return np.arange(n_seqs * self.blocks_per_seq, dtype=np.int32).reshape(n_seqs, self.blocks_per_seq)

    def decode_run(self, batch, ctx, steps, warm):
        """Prefill `batch` sequences one call each, then decode them together so that they
        end near context `ctx`; returns milliseconds per timed decode step."""
        rng = np.random.default_rng(1)
        plen = ctx - (steps + warm) - 2
        tables = self.tables(batch)
        nxt = np.zeros(batch, np.int32)
        for s in range(batch):
            ids = rng.integers(0, self.vocab, plen, dtype=np.int32)
            logits = self.forward(ids, [plen], [0], tables[s:s + 1])
            nxt[s] = int(np.argmax(logits[0]))
        pos = np.full(batch, plen, np.int32)

        def step():
            nonlocal nxt, pos
            logits = self.forward(nxt, np.ones(batch, np.int32), pos, tables)
            nxt = np.argmax(logits, axis=1).astype(np.int32)       # greedy, on the host as the Go engine does
            pos = pos + 1

        for _ in range(warm):
            step()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        return (time.perf_counter() - t0) * 1e3 / steps

    def prefill_run(self, T):
        rng = np.random.default_rng(2)
        ids = rng.integers(0, self.vocab, T, dtype=np.int32)
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            self.forward(ids, [T], [0], self.tables(1))
            ms = (time.perf_counter() - t0) * 1e3
            best = ms if best is None else min(best, ms)
        return best
