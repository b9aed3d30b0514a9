"""Each part alone, built from its PartSpec with weights bound from a dict, against
the plain formulas; a model whose layers differ, run twice or share a cache; and a
toy architecture with a stateful mixer of its own, defined here and registered
without touching the framework."""
import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from plain import llama_plain as plain

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def close(got, want, dtype, what=""):
    got = got.detach().float().cpu().numpy().astype(np.float64)
    scale = max(1e-9, np.abs(want).max())
    err = np.abs(got - want).max()
    assert err <= TOL[dtype] * scale, f"{what}: {err:.3e} > {TOL[dtype]:.0e} * {scale:.3e}"


def stored(a, dtype):
    return (plain.round_bf16(a) if dtype == "bfloat16" else np.asarray(a, np.float32)).astype(np.float64)


def env_for(dtype, hidden, max_position=64):
    from kllm_b200.parts.spec import BuildEnv
    return BuildEnv(dtype=DT[dtype], device=torch.device("cuda"), hidden_size=hidden, max_position=max_position)


def bind(part, weights, dtype):
    tensors = {}
    for s in part.tensor_specs():
        if s.name in weights:
            t = torch.from_numpy(weights[s.name]).cuda()
            tensors[s.name] = t.to(DT[dtype]) if s.store == "compute" else t
    part.bind(tensors)


def one_request_context(n, start=0):
    """A StepContext of one request bringing n tokens at positions start.., with a
    block table over pages 0..; built through the real cache manager."""
    from kllm_b200.parts.context import StepContext
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    return StepContext(n_tokens=n, n_requests=1, token_ids=i32([0] * n), positions=i32(list(range(start, start + n))),
                       token_req=i32([0] * n), q_start=i32([0, n]), start_pos=i32([start]), ctx_len=i32([start + n]),
                       state_slots=i32([0]), block_tables={}, want_rows=i32(list(range(n))), n_want=n,
                       host_n_new=[n], host_start_pos=[start], max_new=n, max_ctx=start + n, all_single=n == 1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    from kllm_b200.parts.spec import PartSpec, part_factory
    rng = np.random.default_rng(0)
    d = 72
    part = part_factory("norm", "rmsnorm")(PartSpec("rmsnorm", "n", {"width": d, "eps": 1e-3}), env_for(dtype, d))
    gain = (1 + 0.2 * rng.standard_normal(d)).astype(np.float32)
    bind(part, {"n.weight": gain}, dtype)
    assert part.gain.dtype == torch.float32
    x0 = rng.standard_normal((5, d)).astype(np.float32)
    res = rng.standard_normal((5, d)).astype(np.float32)
    x = torch.from_numpy(x0).cuda()
    out = part.forward(x, torch.from_numpy(res).cuda().to(DT[dtype]))
    assert out.dtype == DT[dtype]
    close(out, plain.rmsnorm(x0 + stored(res, dtype), gain, 1e-3), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(dtype):
    from kllm_b200.parts.spec import PartSpec, part_factory
    rng = np.random.default_rng(1)
    d, f = 40, 108
    part = part_factory("feed_forward", "gated_mlp")(
        PartSpec("gated_mlp", "ff", {"hidden": d, "intermediate": f, "activation": "silu"}), env_for(dtype, d))
    w = {f"ff.{k}_proj.weight": (rng.standard_normal(s) * 0.3).astype(np.float32)
         for k, s in (("gate", (f, d)), ("up", (f, d)), ("down", (d, f)))}
    bind(part, w, dtype)
    x = rng.standard_normal((7, d)).astype(np.float32)
    out = part.forward(torch.from_numpy(x).cuda().to(DT[dtype]), None)
    rnd = plain.round_act_bf16 if dtype == "bfloat16" else (lambda a: a)
    ws = {k: stored(v, dtype) for k, v in w.items()}
    want = plain.swiglu(stored(x, dtype), ws["ff.gate_proj.weight"], ws["ff.up_proj.weight"],
                        ws["ff.down_proj.weight"], rnd)
    close(out, want, dtype)
    # the route generation takes: the part reads the float32 residual stream, applies the
    # norm itself and adds its result (7 rows: weight-streaming products in bfloat16;
    # 40 rows: library products); both must equal norm -> forward -> sum
    norm = part_factory("norm", "rmsnorm")(PartSpec("rmsnorm", "n", {"width": d, "eps": 1e-5}), env_for(dtype, d))
    gain = (1 + 0.2 * rng.standard_normal(d)).astype(np.float32)
    bind(norm, {"n.weight": gain}, dtype)
    for n in (7, 40):
        x0 = rng.standard_normal((n, d)).astype(np.float32)
        xr = torch.from_numpy(x0).cuda()
        assert part.forward_residual(xr, norm, None) is True
        xn = rnd(plain.rmsnorm(x0, gain, 1e-5))
        close(xr, x0 + plain.swiglu(xn, ws["ff.gate_proj.weight"], ws["ff.up_proj.weight"], ws["ff.down_proj.weight"], rnd),
              dtype, f"residual stream after forward_residual, {n} rows")
    with pytest.raises(ValueError, match="activation"):
        part_factory("feed_forward", "gated_mlp")(
            PartSpec("gated_mlp", "ff", {"hidden": d, "intermediate": f, "activation": "relu"}), env_for(dtype, d))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [None, 6])
def test_attention_part_in_two_portions(dtype, window):
    from kllm_b200.cache import CacheManager
    from kllm_b200.parts.spec import PartSpec, part_factory
    rng = np.random.default_rng(2)
    d, H, G, hd, n = 48, 6, 3, 16, 21
    spec = PartSpec("paged_attention", "a", {
        "hidden": d, "n_heads": H, "n_kv_heads": G, "head_dim": hd, "window": window,
        "position": PartSpec("rotary", "", {"head_dim": hd, "theta": 777.0})})
    part = part_factory("mixer", "paged_attention")(spec, env_for(dtype, d))
    w = {f"a.{k}_proj.weight": (rng.standard_normal(s) * 0.4).astype(np.float32)
         for k, s in (("q", (H * hd, d)), ("k", (G * hd, d)), ("v", (G * hd, d)), ("o", (d, H * hd)))}
    bind(part, w, dtype)
    cache = CacheManager([part.cache_need()], page_size=4, num_pages=9, max_requests=2, dtype=DT[dtype], device="cuda")
    assert cache.groups[0].window == window
    req = cache.open()
    x = rng.standard_normal((n, d)).astype(np.float32)
    xt = torch.from_numpy(x).cuda().to(DT[dtype])
    outs, start = [], 0
    for cnt in (13, 8):
        cache.reserve(req, cnt)
        ctx = one_request_context(cnt, start)
        table = torch.full((1, 8), -1, dtype=torch.int32)
        table[0, :len(req.tables[0])] = torch.tensor(req.tables[0])
        lc = cache.layer_caches({0: table.cuda()})[0]
        outs.append(part.forward(xt[start:start + cnt], ctx, lc))
        cache.commit(req, cnt)
        start += cnt
    cfg = {"head_dim": hd, "num_attention_heads": H, "num_key_value_heads": G, "rope_theta": 777.0,
           "sliding_window": window}
    ws = {"L.self_attn." + k[2:]: stored(v, dtype) for k, v in w.items()}
    rnd = plain.round_act_bf16 if dtype == "bfloat16" else (lambda a: a)
    want = plain.attention_block(stored(x, dtype), ws, "L", cfg, np.arange(n), rnd)
    close(torch.cat(outs), want, dtype)
    if window:
        assert req.tables[0][0] == -1          # the window has passed the first page
    # the route generation takes: the part reads the float32 residual stream, applies the
    # norm in its first kernel and adds its result; a portion of 13 tokens (library
    # products), then 8 single tokens (weight-streaming products and, in bfloat16 with a
    # head size that is a multiple of 32, the fused decode kernel; here the separate ones)
    norm = part_factory("norm", "rmsnorm")(PartSpec("rmsnorm", "n", {"width": d, "eps": 1e-5}), env_for(dtype, d))
    gain = (1 + 0.2 * rng.standard_normal(d)).astype(np.float32)
    bind(norm, {"n.weight": gain}, dtype)
    cache.close(req)
    req2 = cache.open()
    xs, start = torch.from_numpy(x).cuda().clone(), 0
    for cnt in [13] + [1] * 8:
        cache.reserve(req2, cnt)
        ctx = one_request_context(cnt, start)
        table = torch.full((1, 8), -1, dtype=torch.int32)
        table[0, :len(req2.tables[0])] = torch.tensor(req2.tables[0])
        lc = cache.layer_caches({0: table.cuda()})[0]
        assert part.forward_residual(xs[start:start + cnt], norm, ctx, lc) is True
        cache.commit(req2, cnt)
        start += cnt
    xn = rnd(plain.rmsnorm(x, gain, 1e-5))
    close(xs, x + plain.attention_block(xn, ws, "L", cfg, np.arange(n), rnd), dtype, "forward_residual")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(dtype):
    from kllm_b200.parts.spec import PartSpec, part_factory
    rng = np.random.default_rng(3)
    V, d = 53, 24
    table = rng.standard_normal((V, d)).astype(np.float32)
    emb = part_factory("embedding", "token_embedding")(PartSpec("token_embedding", "e", {"vocab": V, "width": d}), env_for(dtype, d))
    head = part_factory("head", "linear_head")(PartSpec("linear_head", "h", {"vocab": V, "width": d, "tied_to": "e.weight"}), env_for(dtype, d))
    t = {"e.weight": torch.from_numpy(table).cuda().to(DT[dtype])}
    emb.bind(t)
    head.bind(t)
    ids = torch.tensor([52, 0, 7], dtype=torch.int32, device="cuda")
    x = emb.forward(ids)
    assert x.dtype == torch.float32 and np.array_equal(x.cpu().numpy().astype(np.float64), stored(table, dtype)[[52, 0, 7]])
    logits = head.forward(x.to(DT[dtype]))
    assert logits.dtype == torch.float32
    close(logits, stored(table, dtype)[[52, 0, 7]] @ stored(table, dtype).T, dtype)


@pytest.mark.parametrize("n", [6, 12])
def test_feed_forward_part_fused_route_with_a_width_that_needs_slices(n):
    """The decode route (norm inside the gate/up kernel, down product adding into the
    residual stream) with an intermediate width too long for the down kernel's shared
    memory at 12 rows: that product runs over column slices."""
    from kllm_b200 import kernels
    from kllm_b200.parts.spec import PartSpec, part_factory
    rng = np.random.default_rng(n)
    d, f = 64, 6016
    assert not kernels.skinny_fits(12, f, torch.bfloat16) and kernels.skinny_fits(6, f, torch.bfloat16)
    env = env_for("bfloat16", d)
    part = part_factory("feed_forward", "gated_mlp")(
        PartSpec("gated_mlp", "ff", {"hidden": d, "intermediate": f, "activation": "silu"}), env)
    norm = part_factory("norm", "rmsnorm")(PartSpec("rmsnorm", "n", {"width": d, "eps": 1e-5}), env)
    w = {f"ff.{k}_proj.weight": (rng.standard_normal(s) * 0.05).astype(np.float32)
         for k, s in (("gate", (f, d)), ("up", (f, d)), ("down", (d, f)))}
    w["ff.down_proj.weight"][:, f - 1] = 0.5          # the last column of the last slice counts
    gain = (1 + 0.2 * rng.standard_normal(d)).astype(np.float32)
    bind(part, w, "bfloat16")
    bind(norm, {"n.weight": gain}, "bfloat16")
    x0 = rng.standard_normal((n, d)).astype(np.float32)
    x = torch.from_numpy(x0).cuda()
    assert part.forward_residual(x, norm, None) is True
    ws = {k: stored(v, "bfloat16") for k, v in w.items()}
    xn = plain.round_act_bf16(plain.rmsnorm(x0, gain, 1e-5))
    want = x0 + plain.swiglu(xn, ws["ff.gate_proj.weight"], ws["ff.up_proj.weight"], ws["ff.down_proj.weight"],
                             plain.round_act_bf16)
    close(x, want, "bfloat16", "residual stream after the fused feed-forward")
    kernels.check_status("cuda")


@pytest.mark.parametrize("n", [40, 300])
def test_feed_forward_part_on_the_tensor_core_route(n, monkeypatch):
    """The gated feed-forward with gate, up and activation in one tcgen05 kernel, the
    route of large portions, forced here for a small one."""
    from kllm_b200 import kernels
    from kllm_b200.parts.spec import PartSpec, part_factory
    rng = np.random.default_rng(9)
    d, f = 72, 200
    part = part_factory("feed_forward", "gated_mlp")(
        PartSpec("gated_mlp", "mlp", {"hidden": d, "intermediate": f, "activation": "silu"}), env_for("bfloat16", d))
    w = {f"mlp.{k}_proj.weight": (rng.standard_normal(shape) * 0.1).astype(np.float32)
         for k, shape in (("gate", (f, d)), ("up", (f, d)), ("down", (d, f)))}
    bind(part, w, "bfloat16")
    xn = rng.standard_normal((n, d)).astype(np.float32)
    xt = torch.from_numpy(xn).cuda().to(torch.bfloat16)
    monkeypatch.setattr(kernels, "gemm_pays", lambda *a, **k: False)
    library = part.forward(xt, None)
    monkeypatch.setattr(kernels, "gemm_pays", lambda *a, **k: True)
    calls, real_gemm = [], kernels.gemm
    monkeypatch.setattr(kernels, "gemm", lambda *a, **k: calls.append(k.get("epilogue")) or real_gemm(*a, **k))
    fused = part.forward(xt, None)
    assert calls == ["swiglu"]
    xs = stored(xn, "bfloat16")
    g, u = xs @ stored(w["mlp.gate_proj.weight"], "bfloat16").T, xs @ stored(w["mlp.up_proj.weight"], "bfloat16").T
    want = plain.round_act_bf16(plain.silu(g) * u) @ stored(w["mlp.down_proj.weight"], "bfloat16").T
    close(fused, want, "bfloat16", "fused route")
    close(library, want, "bfloat16", "library route")
    kernels.check_status("cuda")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rotary_dim", [None, 8])
def test_rotary_part_rotates_and_stores(dtype, rotary_dim):
    """The position part alone: q rotated in place, rotated k and v stored at the
    pages' slots; a partial rotary width leaves the other dims alone."""
    from kllm_b200.cache import CacheManager
    from kllm_b200.parts.spec import PagedKVNeed, PartSpec, part_factory
    rng = np.random.default_rng(7)
    H, G, hd, n, start = 3, 1, 16, 9, 5
    params = {"head_dim": hd, "theta": 50.0}
    if rotary_dim:
        params["rotary_dim"] = rotary_dim
    part = part_factory("position", "rotary")(PartSpec("rotary", "", params), env_for(dtype, 48))
    rot = rotary_dim or hd
    assert (part.full_rotary_table() is None) == (rot != hd)
    cache = CacheManager([PagedKVNeed(G, hd)], page_size=4, num_pages=6, max_requests=1, dtype=DT[dtype], device="cuda")
    req = cache.open()
    cache.reserve(req, start + n)
    cache.commit(req, start)
    qkv = rng.standard_normal((n, (H + 2 * G) * hd)).astype(np.float32)
    t = torch.from_numpy(qkv).cuda().to(DT[dtype])
    q, k, v = t[:, :H * hd], t[:, H * hd:(H + G) * hd], t[:, (H + G) * hd:]
    ctx = one_request_context(n, start)
    table = torch.tensor([req.tables[0]], dtype=torch.int32, device="cuda")
    lc = cache.layer_caches({0: table})[0]
    part.apply(q, k, v, ctx, lc, H, G)
    sq = stored(qkv, dtype)
    pos = np.arange(start, start + n)

    def rotated(x, heads):
        x = x.reshape(n, heads, hd).copy()
        x[:, :, :rot] = plain.rope(x[:, :, :rot].reshape(n, heads * rot), pos, heads, rot, 50.0).reshape(n, heads, rot)
        return x.reshape(n, heads * hd)

    close(q, rotated(sq[:, :H * hd], H), dtype, "q")
    kw = rotated(sq[:, H * hd:(H + G) * hd], G).reshape(n, G, hd)
    for i, p_ in enumerate(pos):
        pg, slot = req.tables[0][p_ // 4], p_ % 4
        close(lc.k[pg, :, slot], kw[i], dtype, f"k at position {p_}")
        close(lc.v[pg, :, slot], sq[i, (H + G) * hd:].reshape(G, hd), dtype, f"v at position {p_}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n", [3, 40])
def test_block_part_both_routes(dtype, n):
    """A whole pre-norm block against the plain layer.  Both sizes go through the parts'
    ``forward_residual`` as in generation: n = 3 with the norm and the residual sum inside
    weight-streaming products (bfloat16), n = 40 with the norm kernel, library products and
    the sum in the last product's epilogue.  The route norm -> ``forward`` -> pending is
    what parts without ``forward_residual`` get (the toy mixers below)."""
    from kllm_b200.cache import CacheManager
    from kllm_b200.parts.spec import BlockSpec, PartSpec, part_factory
    rng = np.random.default_rng(8)
    d, H, G, hd, f = 64, 4, 2, 16, 96
    norm = {"width": d, "eps": 1e-5}
    spec = BlockSpec("pre_norm", "model.layers.0",
                     PartSpec("paged_attention", "model.layers.0.self_attn", {
                         "hidden": d, "n_heads": H, "n_kv_heads": G, "head_dim": hd, "window": None,
                         "position": PartSpec("rotary", "", {"head_dim": hd, "theta": 1e4})}),
                     PartSpec("gated_mlp", "model.layers.0.mlp", {"hidden": d, "intermediate": f, "activation": "silu"}),
                     PartSpec("rmsnorm", "model.layers.0.input_layernorm", dict(norm)),
                     PartSpec("rmsnorm", "model.layers.0.post_attention_layernorm", dict(norm)))
    block = part_factory("block", "pre_norm")(spec, env_for(dtype, d))
    cfg = {"num_hidden_layers": 1, "hidden_size": d, "num_attention_heads": H, "num_key_value_heads": G, "head_dim": hd,
           "intermediate_size": f, "vocab_size": 8, "rope_theta": 1e4, "rms_norm_eps": 1e-5}
    w = plain.random_weights(cfg, 3, gain_std=0.1, std=0.15)
    bind(block, w, dtype)
    cache = CacheManager([block.mixer.cache_need()], page_size=16, num_pages=4, max_requests=1, dtype=DT[dtype], device="cuda")
    req = cache.open()
    cache.reserve(req, n)
    x0 = rng.standard_normal((n, d)).astype(np.float32)
    x = torch.from_numpy(x0).cuda()
    ctx = one_request_context(n, 0)
    table = torch.tensor([req.tables[0]], dtype=torch.int32, device="cuda")
    pending = block.forward(x, None, ctx, cache.layer_caches({0: table})[0])
    got = x if pending is None else x + pending.float()
    ws = {k: (stored(v, dtype) if v.ndim == 2 else v) for k, v in w.items()}
    rnd = plain.round_act_bf16 if dtype == "bfloat16" else (lambda a: a)
    want = plain.decoder_layer(x0.astype(np.float64), ws, 0, plain.normalise_config(cfg), np.arange(n), rnd)
    close(got, want, dtype, f"block output, {n} tokens")
    assert pending is None, "both parts add into the residual stream themselves"


# ---- a toy architecture defined in the test -----------------------------------

class RunningMeanMixer:
    """out_t = W . mean(x_0..x_t): needs the sum of a request's inputs so far and
    their count, i.e. per-request state of fixed size, and no pages.  It reads slot
    numbers on the host, so it asks not to be captured into a CUDA graph."""

    graph_safe = False

    def __init__(self, spec, env):
        self.d = spec.params["hidden"]
        self.name = spec.prefix + ".mix.weight"
        self.dtype = env.dtype

    def tensor_specs(self):
        from kllm_b200.parts.spec import TensorSpec
        return [TensorSpec(self.name, (self.d, self.d))]

    def bind(self, tensors):
        self.w = tensors[self.name]

    def cache_need(self):
        from kllm_b200.parts.spec import StateNeed
        return StateNeed((self.d + 1,), "float32")

    def forward(self, xn, ctx, cache):
        out = torch.empty_like(xn)
        row = 0
        slots = ctx.state_slots.tolist()
        for s, n in enumerate(ctx.host_n_new):
            st = cache.state[slots[s]]
            x = xn[row:row + n].float()
            sums = st[:self.d] + torch.cumsum(x, dim=0)
            counts = st[self.d] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
            out[row:row + n] = ((sums / counts[:, None]) @ self.w.float().t()).to(self.dtype)
            st[:self.d] = sums[-1]
            st[self.d] = counts[-1]
            row += n
        return out


def toy_spec(cfg):
    from kllm_b200.parts.spec import BlockSpec, LayerCall, ModelSpec, PartSpec
    d = cfg.hidden
    norm = {"width": d, "eps": 1e-5}
    rotary = PartSpec("rotary", "", {"head_dim": 16, "theta": 100.0})
    ff = lambda p: PartSpec("gated_mlp", p + ".mlp", {"hidden": d, "intermediate": 2 * d, "activation": "silu"})
    blocks = [
        BlockSpec("pre_norm", "layers.0", PartSpec("toy_running_mean", "layers.0", {"hidden": d}), ff("layers.0"),
                  PartSpec("rmsnorm", "layers.0.n1", dict(norm)), PartSpec("rmsnorm", "layers.0.n2", dict(norm))),
        BlockSpec("pre_norm", "layers.1", PartSpec("paged_attention", "layers.1.attn", {
            "hidden": d, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16, "window": None, "position": rotary}),
            ff("layers.1"), PartSpec("rmsnorm", "layers.1.n1", dict(norm)), PartSpec("rmsnorm", "layers.1.n2", dict(norm))),
    ]
    # layer 0, layer 1, layer 0 again with a state of its own, layer 1 again reading the keys it wrote before
    schedule = [LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(1, 1, writes_cache=False)]
    return ModelSpec(hidden_size=d, vocab_size=cfg.vocab, max_position=64,
                     embedding=PartSpec("token_embedding", "emb", {"vocab": cfg.vocab, "width": d}),
                     blocks=blocks, schedule=schedule, final_norm=PartSpec("rmsnorm", "final", dict(norm)),
                     head=PartSpec("linear_head", "head", {"vocab": cfg.vocab, "width": d, "tied_to": "emb.weight"}))


def plain_toy(w, ids, d):
    """The toy model on whole sequences, in float64, without any cache."""
    n = len(ids)
    x = plain.embed(w["emb.weight"], ids)

    def layer0(x):
        xn = plain.rmsnorm(x, w["layers.0.n1.weight"], 1e-5)
        mean = np.cumsum(xn, 0) / np.arange(1, n + 1)[:, None]
        x = x + mean @ plain.f64(w["layers.0.mix.weight"]).T
        xn = plain.rmsnorm(x, w["layers.0.n2.weight"], 1e-5)
        return x + plain.swiglu(xn, w["layers.0.mlp.gate_proj.weight"], w["layers.0.mlp.up_proj.weight"],
                                w["layers.0.mlp.down_proj.weight"])

    def layer1(x, kv=None):
        xn = plain.rmsnorm(x, w["layers.1.n1.weight"], 1e-5)
        p = "layers.1.attn."
        q = plain.rope(xn @ plain.f64(w[p + "q_proj.weight"]).T, np.arange(n), 2, 16, 100.0)
        if kv is None:
            k = plain.rope(xn @ plain.f64(w[p + "k_proj.weight"]).T, np.arange(n), 1, 16, 100.0)
            kv = (k, xn @ plain.f64(w[p + "v_proj.weight"]).T)
        x = x + plain.attention(q, kv[0], kv[1], 2, 1, 16) @ plain.f64(w[p + "o_proj.weight"]).T
        xn = plain.rmsnorm(x, w["layers.1.n2.weight"], 1e-5)
        return x + plain.swiglu(xn, w["layers.1.mlp.gate_proj.weight"], w["layers.1.mlp.up_proj.weight"],
                                w["layers.1.mlp.down_proj.weight"]), kv

    x = layer0(x)
    x, kv = layer1(x)
    x = layer0(x)
    x, _ = layer1(x, kv)
    return plain.rmsnorm(x, w["final.weight"], 1e-5) @ plain.f64(w["emb.weight"]).T


def test_toy_architecture_with_a_stateful_mixer(tmp_path):
    """Registered, built, loaded and stepped through the unchanged framework: parts
    registry, architecture registry, loader, cache manager (state slots beside
    pages), step function with portions and two live requests."""
    import json
    from kllm_b200.config import ModelConfig, register_architecture
    from kllm_b200.engine import Engine, Options, StepEntry
    from kllm_b200.parts.spec import register_part
    from kllm_b200.weights import save_tensors

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        hidden: int = 32
        vocab: int = 40

        @classmethod
        def from_dict(cls, d):
            return cls(architecture=d["architectures"][0], hidden=d["hidden"], vocab=d["vocab"])

    register_part("mixer", "toy_running_mean", RunningMeanMixer)
    register_architecture("ToyRunningMeanLM", ToyConfig, toy_spec)

    d = 32
    rng = np.random.default_rng(4)
    mat = lambda r, c: (rng.standard_normal((r, c)) * 0.25).astype(np.float32)
    w = {"emb.weight": mat(40, d), "final.weight": np.ones(d, np.float32)}
    for l in (0, 1):
        w.update({f"layers.{l}.n1.weight": (1 + 0.1 * rng.standard_normal(d)).astype(np.float32),
                  f"layers.{l}.n2.weight": np.ones(d, np.float32),
                  f"layers.{l}.mlp.gate_proj.weight": mat(2 * d, d), f"layers.{l}.mlp.up_proj.weight": mat(2 * d, d),
                  f"layers.{l}.mlp.down_proj.weight": mat(d, 2 * d)})
    w["layers.0.mix.weight"] = mat(d, d)
    w.update({"layers.1.attn.q_proj.weight": mat(32, d) * 4, "layers.1.attn.k_proj.weight": mat(16, d) * 4,
              "layers.1.attn.v_proj.weight": mat(16, d), "layers.1.attn.o_proj.weight": mat(d, 32)})
    model_dir = tmp_path / "toy"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps({"architectures": ["ToyRunningMeanLM"], "hidden": d, "vocab": 40}))
    save_tensors(str(model_dir / "model.safetensors"), {k: torch.from_numpy(v) for k, v in w.items()})

    eng = Engine(str(model_dir), Options(dtype="float32", max_seq=64, block_size=4, num_blocks=12, max_batch=2))
    assert eng.model.n_cache_slots == 3 and len(eng.cache.groups) == 1 and sorted(eng.cache.state) == [0, 2]
    a_ids = rng.integers(0, 40, 19).tolist()
    b_ids = rng.integers(0, 40, 11).tolist()
    a, b = eng.cache.open(), eng.cache.open()
    got_a, got_b = [], []
    # a: 7 | 1 | 9 | 2 ; b joins later: 4 | 6 | 1
    l1 = eng.step([StepEntry(a, a_ids[:7], range(7))]); got_a.append(l1)
    l2 = eng.step([StepEntry(a, a_ids[7:8], [0]), StepEntry(b, b_ids[:4], range(4))]); got_a.append(l2[:1]); got_b.append(l2[1:])
    l3 = eng.step([StepEntry(b, b_ids[4:10], range(6)), StepEntry(a, a_ids[8:17], range(9))]); got_b.append(l3[:6]); got_a.append(l3[6:])
    l4 = eng.step([StepEntry(a, a_ids[17:], range(2)), StepEntry(b, b_ids[10:], [0])]); got_a.append(l4[:2]); got_b.append(l4[2:])
    close(torch.cat(got_a), plain_toy(w, a_ids, d), "float32", "request a")
    close(torch.cat(got_b), plain_toy(w, b_ids, d), "float32", "request b")
    assert not eng.runner.use_graphs, "a part that is not graph-safe keeps decode steps out of CUDA graphs"
    # a new request in a's slot starts from zero state
    eng.cache.close(a)
    c = eng.cache.open()
    assert c.state_slot == a.state_slot
    close(eng.step([StepEntry(c, b_ids, range(11))]), plain_toy(w, b_ids, d), "float32", "reused state slot")
    eng.close()


# ---- toy parts of the other families: a routed feed-forward, another position encoding ----

class TopOneExperts:
    """out = p_e . (W_e x) for the expert e with the largest router probability
    (softmax over the router's float32 logits): a feed-forward with routing."""

    def __init__(self, spec, env):
        self.d, self.n = spec.params["hidden"], spec.params["experts"]
        self.p = spec.prefix
        self.dtype = env.dtype

    def tensor_specs(self):
        from kllm_b200.parts.spec import TensorSpec
        return [TensorSpec(self.p + ".router.weight", (self.n, self.d), store="float32")] + \
               [TensorSpec(f"{self.p}.experts.{e}.weight", (self.d, self.d)) for e in range(self.n)]

    def bind(self, tensors):
        self.router = tensors[self.p + ".router.weight"]
        self.experts = [tensors[f"{self.p}.experts.{e}.weight"] for e in range(self.n)]

    def forward(self, xn, ctx):
        prob = torch.softmax(xn.float() @ self.router.t(), dim=-1)
        top_p, top_e = prob.max(dim=-1)
        out = torch.zeros((xn.shape[0], self.d), dtype=torch.float32, device=xn.device)
        for e in range(self.n):          # every expert on every row, the others masked: shapes that a graph can replay
            gate = torch.where(top_e == e, top_p, torch.zeros_like(top_p))
            out += gate[:, None] * (xn.float() @ self.experts[e].float().t())
        return out


class HalfSpeedRotary:
    """Rotary encoding whose angle grows with position / 2 (positions interpolated): a
    position part with a table of its own, through the same kernels as the built-in one."""

    def __init__(self, spec, env):
        hd = self.head_dim = spec.params["head_dim"]
        j = torch.arange(hd // 2, dtype=torch.float64)
        ang = (torch.arange(env.max_position, dtype=torch.float64) / 2.0)[:, None] * torch.pow(
            torch.tensor(float(spec.params["theta"]), dtype=torch.float64), -2.0 * j / hd)[None, :]
        self.cos_sin = torch.cat([torch.cos(ang), torch.sin(ang)], dim=1).to(torch.float32).contiguous().to(env.device)

    def tensor_specs(self):
        return []

    def bind(self, tensors):
        pass

    def full_rotary_table(self):
        return self.cos_sin

    def apply(self, q, k, v, ctx, cache, n_heads, n_kv_heads):
        from kllm_b200 import kernels
        kernels.rope_append(q, k, v, self.cos_sin, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.v,
                            n_heads, n_kv_heads, self.head_dim)


def routed_spec(cfg):
    from kllm_b200.parts.spec import BlockSpec, LayerCall, ModelSpec, PartSpec
    d = cfg.hidden
    norm = {"width": d, "eps": 1e-6}
    pos = PartSpec("toy_half_speed_rotary", "", {"head_dim": 32, "theta": 50.0})
    blocks = [BlockSpec("pre_norm", f"l.{i}",
                        PartSpec("paged_attention", f"l.{i}.attn", {"hidden": d, "n_heads": 2, "n_kv_heads": 2, "head_dim": 32,
                                                                   "window": 6 if i == 1 else None, "position": pos}),
                        PartSpec("toy_top_one_experts", f"l.{i}.moe", {"hidden": d, "experts": 3}),
                        PartSpec("rmsnorm", f"l.{i}.n1", dict(norm)), PartSpec("rmsnorm", f"l.{i}.n2", dict(norm)))
              for i in range(2)]
    return ModelSpec(hidden_size=d, vocab_size=cfg.vocab, max_position=64,
                     embedding=PartSpec("token_embedding", "emb", {"vocab": cfg.vocab, "width": d}),
                     blocks=blocks, schedule=[LayerCall(0, 0), LayerCall(1, 1)],
                     final_norm=PartSpec("rmsnorm", "final", dict(norm)),
                     head=PartSpec("linear_head", "head", {"vocab": cfg.vocab, "width": d, "tied_to": None}))


def plain_routed(w, ids, d, rnd=lambda a: a):
    n = len(ids)
    x = plain.embed(w["emb.weight"], ids)
    pos = np.arange(n) / 2.0
    for i in range(2):
        p = f"l.{i}.attn."
        xn = rnd(plain.rmsnorm(x, w[f"l.{i}.n1.weight"], 1e-6))
        q = rnd(plain.rope(rnd(xn @ plain.f64(w[p + "q_proj.weight"]).T), pos, 2, 32, 50.0))
        k = rnd(plain.rope(rnd(xn @ plain.f64(w[p + "k_proj.weight"]).T), pos, 2, 32, 50.0))
        v = rnd(xn @ plain.f64(w[p + "v_proj.weight"]).T)
        att = rnd(plain.attention(q, k, v, 2, 2, 32, window=6 if i == 1 else None,
                                  rnd_p=None if rnd(np.float64(1 / 3)) == 1 / 3 else plain.round_act_bf16))
        x = x + att @ plain.f64(w[p + "o_proj.weight"]).T
        xn = rnd(plain.rmsnorm(x, w[f"l.{i}.n2.weight"], 1e-6))
        logits = xn @ plain.f64(w[f"l.{i}.moe.router.weight"]).T
        prob = np.exp(logits - logits.max(-1, keepdims=True))
        prob /= prob.sum(-1, keepdims=True)
        e = prob.argmax(-1)
        out = np.stack([prob[t, e[t]] * (xn[t] @ plain.f64(w[f"l.{i}.moe.experts.{e[t]}.weight"]).T) for t in range(n)])
        x = x + out
    return plain.rmsnorm(x, w["final.weight"], 1e-6) @ plain.f64(w["head.weight"]).T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_routed_experts_and_its_own_position_encoding(tmp_path, dtype):
    """A feed-forward with routing and a position encoding that the framework does not
    have, registered from here; whole prompts, portions, and tokens one by one (which
    takes the decode attention kernel with the toy part's table) agree with the plain
    sum.  One layer has a window, so the cache manager keeps two groups of pages."""
    import json
    from kllm_b200.config import ModelConfig, register_architecture
    from kllm_b200.engine import Engine, Options, StepEntry
    from kllm_b200.parts.spec import register_part
    from kllm_b200.weights import save_tensors

    @dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        hidden: int = 64
        vocab: int = 48

        @classmethod
        def from_dict(cls, d):
            return cls(architecture=d["architectures"][0], hidden=d["hidden"], vocab=d["vocab"])

    register_part("feed_forward", "toy_top_one_experts", TopOneExperts)
    register_part("position", "toy_half_speed_rotary", HalfSpeedRotary)
    register_architecture("ToyRoutedLM", RoutedConfig, routed_spec)

    d = 64
    rng = np.random.default_rng(11)
    mat = lambda r, c, s=0.2: (rng.standard_normal((r, c)) * s).astype(np.float32)
    w = {"emb.weight": mat(48, d, 1.0), "head.weight": mat(48, d), "final.weight": np.ones(d, np.float32)}
    for i in range(2):
        w.update({f"l.{i}.n1.weight": (1 + 0.1 * rng.standard_normal(d)).astype(np.float32),
                  f"l.{i}.n2.weight": np.ones(d, np.float32),
                  f"l.{i}.attn.q_proj.weight": mat(64, d, 0.4), f"l.{i}.attn.k_proj.weight": mat(64, d, 0.4),
                  f"l.{i}.attn.v_proj.weight": mat(64, d), f"l.{i}.attn.o_proj.weight": mat(d, 64),
                  f"l.{i}.moe.router.weight": mat(3, d, 1.5)})      # far apart: no routing decision near a tie
        w.update({f"l.{i}.moe.experts.{e}.weight": mat(d, d) for e in range(3)})
    model_dir = tmp_path / "routed"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps({"architectures": ["ToyRoutedLM"], "hidden": d, "vocab": 48}))
    store = lambda k, v: torch.from_numpy(v) if (v.ndim == 1 or "router" in k or dtype == "float32") \
        else torch.from_numpy(v).to(torch.bfloat16)
    save_tensors(str(model_dir / "model.safetensors"), {k: store(k, v) for k, v in w.items()})
    ws = {k: (v if (v.ndim == 1 or "router" in k) else stored(v, dtype)) for k, v in w.items()}
    rnd = plain.round_act_bf16 if dtype == "bfloat16" else (lambda a: a)

    eng = Engine(str(model_dir), Options(dtype=dtype, max_seq=64, block_size=4, num_blocks=40, max_batch=2))
    assert len(eng.cache.groups) == 2, "a full and a windowed group of pages"
    ids = rng.integers(0, 48, 37).tolist()
    want = plain_routed(ws, ids, d, rnd)
    a = eng.cache.open()
    close(eng.step([StepEntry(a, ids, range(37))]), want, dtype, "whole prompt")
    b = eng.cache.open()
    got = [eng.step([StepEntry(b, ids[:9], range(9))]), eng.step([StepEntry(b, ids[9:11], range(2))]),
           eng.step([StepEntry(b, ids[11:30], range(19))])]
    got += [eng.step([StepEntry(b, ids[t:t + 1], [0])]) for t in range(30, 37)]       # one by one
    close(torch.cat(got), want, dtype, "portions, then token by token")
    eng.close()


# ---- a transform of q and k before the position encoding, defined in the test -----------

class HeadRMSNorm:
    """q and k normalised per head with a learned gain each (a "qk-norm"): a part of the
    qk_transform family, registered from here.  Plain torch on the strided views."""

    def __init__(self, spec, env):
        self.prefix, self.hd, self.eps = spec.prefix, spec.params["head_dim"], spec.params["eps"]

    def tensor_specs(self):
        from kllm_b200.parts.spec import TensorSpec
        return [TensorSpec(f"{self.prefix}.q_norm.weight", (self.hd,), store="float32", init="gain"),
                TensorSpec(f"{self.prefix}.k_norm.weight", (self.hd,), store="float32", init="gain")]

    def bind(self, tensors):
        self.gq, self.gk = tensors[f"{self.prefix}.q_norm.weight"], tensors[f"{self.prefix}.k_norm.weight"]

    def apply(self, q, k, ctx, n_heads, n_kv_heads, head_dim):
        for t, g, heads in ((q, self.gq, n_heads), (k, self.gk, n_kv_heads)):
            if t is None:
                continue
            v = t.float().reshape(t.shape[0], heads, head_dim)
            v = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + self.eps) * g
            t.copy_(v.reshape(t.shape[0], heads * head_dim).to(t.dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_part_with_a_qk_transform_registered_from_outside(dtype):
    """The attention part with a per-head norm on q and k between the projection and the
    rotation: a portion of 9 tokens, then 6 single tokens.  Head size 32 in bfloat16 would
    take the fused decode kernel, which rotates the raw projections itself; with a
    transform the part must take the separate kernels, and the answers must be the plain
    formula's with the norm in place."""
    from kllm_b200 import kernels
    from kllm_b200.cache import CacheManager
    from kllm_b200.parts.spec import PartSpec, part_factory, register_part
    register_part("qk_transform", "toy_head_rmsnorm", HeadRMSNorm)
    rng = np.random.default_rng(21)
    d, H, G, hd, n, theta, eps = 64, 4, 2, 32, 15, 300.0, 1e-4
    spec = PartSpec("paged_attention", "a", {
        "hidden": d, "n_heads": H, "n_kv_heads": G, "head_dim": hd,
        "position": PartSpec("rotary", "", {"head_dim": hd, "theta": theta}),
        "qk_transform": PartSpec("toy_head_rmsnorm", "a", {"head_dim": hd, "eps": eps})})
    part = part_factory("mixer", "paged_attention")(spec, env_for(dtype, d))
    assert sorted(s.name for s in part.tensor_specs())[:2] == ["a.k_norm.weight", "a.k_proj.weight"]
    w = {f"a.{k}_proj.weight": (rng.standard_normal(s) * 0.4).astype(np.float32)
         for k, s in (("q", (H * hd, d)), ("k", (G * hd, d)), ("v", (G * hd, d)), ("o", (d, H * hd)))}
    w["a.q_norm.weight"] = (1 + 0.3 * rng.standard_normal(hd)).astype(np.float32)
    w["a.k_norm.weight"] = (1 + 0.3 * rng.standard_normal(hd)).astype(np.float32)
    bind(part, w, dtype)
    norm = part_factory("norm", "rmsnorm")(PartSpec("rmsnorm", "n", {"width": d, "eps": 1e-5}), env_for(dtype, d))
    gain = (1 + 0.2 * rng.standard_normal(d)).astype(np.float32)
    bind(norm, {"n.weight": gain}, dtype)
    cache = CacheManager([part.cache_need()], page_size=4, num_pages=6, max_requests=1, dtype=DT[dtype], device="cuda")
    req = cache.open()
    x = rng.standard_normal((n, d)).astype(np.float32)
    xs, start = torch.from_numpy(x).cuda().clone(), 0
    calls, real = [], kernels.attention_decode_fused
    kernels.attention_decode_fused = lambda *a, **k: calls.append(1) or real(*a, **k)
    try:
        for cnt in [9] + [1] * 6:
            cache.reserve(req, cnt)
            ctx = one_request_context(cnt, start)
            table = torch.full((1, 4), -1, dtype=torch.int32)
            table[0, :len(req.tables[0])] = torch.tensor(req.tables[0])
            assert part.forward_residual(xs[start:start + cnt], norm, ctx, cache.layer_caches({0: table.cuda()})[0])
            cache.commit(req, cnt)
            start += cnt
    finally:
        kernels.attention_decode_fused = real
    assert not calls, "the fused decode kernel cannot apply a transform between projection and rotation"
    rnd = plain.round_act_bf16 if dtype == "bfloat16" else (lambda a: a)
    ws = {k: stored(v, dtype) for k, v in w.items() if v.ndim == 2}
    xn = rnd(plain.rmsnorm(x, gain, 1e-5))

    def head_norm(t, g, heads):
        v = t.reshape(n, heads, hd)
        return rnd((v / np.sqrt((v * v).mean(-1, keepdims=True) + eps) * g).reshape(n, heads * hd))

    q = head_norm(rnd(xn @ ws["a.q_proj.weight"].T), w["a.q_norm.weight"].astype(np.float64), H)
    k = head_norm(rnd(xn @ ws["a.k_proj.weight"].T), w["a.k_norm.weight"].astype(np.float64), G)
    v = rnd(xn @ ws["a.v_proj.weight"].T)
    q, k = rnd(plain.rope(q, np.arange(n), H, hd, theta)), rnd(plain.rope(k, np.arange(n), G, hd, theta))
    att = rnd(plain.attention(q, k, v, H, G, hd, rnd_p=None if dtype == "float32" else rnd))
    close(xs, x + att @ ws["a.o_proj.weight"].T, dtype, "attention with a q/k norm per head")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [None, 300])
def test_attention_part_with_a_bias_on_the_scores_instead_of_a_rotation(dtype, window):
    """A position encoding that acts on the scores: slope[h] * (key position - query position)
    added to the scaled scores, no rotation of q and k.  The part takes the CUDA-core
    attention kernel (the tensor-core kernels have no such argument): a portion of 290
    tokens, then single tokens whose contexts are cut into chunks of 256 keys and merged."""
    from kllm_b200.cache import CacheManager
    from kllm_b200.parts.spec import PartSpec, part_factory
    rng = np.random.default_rng(31)
    d, H, G, hd, n = 64, 4, 2, 32, 300
    slopes = [2.0 ** -(h + 1) for h in range(H)]
    spec = PartSpec("paged_attention", "a", {"hidden": d, "n_heads": H, "n_kv_heads": G, "head_dim": hd, "window": window,
                                             "position": None, "score_slopes": slopes})
    part = part_factory("mixer", "paged_attention")(spec, env_for(dtype, d, max_position=512))
    w = {f"a.{k}_proj.weight": (rng.standard_normal(s) * 0.3).astype(np.float32)
         for k, s in (("q", (H * hd, d)), ("k", (G * hd, d)), ("v", (G * hd, d)), ("o", (d, H * hd)))}
    bind(part, w, dtype)
    cache = CacheManager([part.cache_need()], page_size=16, num_pages=20, max_requests=1, dtype=DT[dtype], device="cuda")
    req = cache.open()
    x = rng.standard_normal((n, d)).astype(np.float32)
    xt = torch.from_numpy(x).cuda().to(DT[dtype])
    outs, start = [], 0
    for cnt in [290] + [1] * 10:
        cache.reserve(req, cnt)
        ctx = one_request_context(cnt, start)
        table = torch.full((1, 20), -1, dtype=torch.int32)
        table[0, :len(req.tables[0])] = torch.tensor(req.tables[0])
        outs.append(part.forward(xt[start:start + cnt], ctx, cache.layer_caches({0: table.cuda()})[0]))
        cache.commit(req, cnt)
        start += cnt
    rnd = plain.round_act_bf16 if dtype == "bfloat16" else (lambda a: a)
    ws = {k: stored(v, dtype) for k, v in w.items()}
    xs = stored(x, dtype)
    q, k, v = (rnd(xs @ ws[f"a.{m}_proj.weight"].T) for m in "qkv")
    pos = np.arange(n)
    mask = pos[:, None] >= pos[None, :]
    if window:
        mask &= pos[None, :] > pos[:, None] - window
    att = np.zeros((n, H * hd))
    for h in range(H):
        g = h // (H // G)
        sc = (q[:, h * hd:(h + 1) * hd] @ k[:, g * hd:(g + 1) * hd].T) / math.sqrt(hd) + slopes[h] * (pos[None, :] - pos[:, None])
        sc = np.where(mask, sc, -np.inf)
        p = np.exp(sc - sc.max(axis=1, keepdims=True))
        att[:, h * hd:(h + 1) * hd] = (p @ v[:, g * hd:(g + 1) * hd]) / p.sum(axis=1, keepdims=True)
    close(torch.cat(outs), rnd(att) @ ws["a.o_proj.weight"].T, dtype, "attention with a bias on the scores")
