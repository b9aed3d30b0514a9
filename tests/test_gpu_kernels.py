"""Each kernel alone against a plain float64 formula, at sizes other than the
tiny models': widths and vocabularies that are no power of two, head sizes in
steps of 16, odd head counts, scattered pages.  Where random numbers would hide a
fault the inputs are made so that it shows: one far key that must win, a key just
outside a window that must not be seen, NaN in every cache slot that must not be
read."""
import math

import numpy as np
import pytest
import torch

from plain import llama_plain as plain

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 1e-5, "bfloat16": 1.6e-2}      # relative to the largest |value|


def dev(a, dtype=None):
    t = torch.as_tensor(np.asarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def close(got, want, dtype, what=""):
    got = got.detach().float().cpu().numpy().astype(np.float64)
    scale = max(1e-9, np.abs(want).max())
    err = np.abs(got - want).max()
    assert err <= TOL[dtype] * scale, f"{what}: {err:.3e} > {TOL[dtype]:.0e} * {scale:.3e}"


def as_stored(a, dtype):
    """What the kernel sees of float32 data stored in the given dtype, as float64."""
    return (plain.round_bf16(a) if dtype == "bfloat16" else np.asarray(a, np.float32)).astype(np.float64)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed_and_gather(dtype):
    from kllm_b200 import kernels
    rng = np.random.default_rng(0)
    table = rng.standard_normal((37, 24)).astype(np.float32)
    ids = np.array([36, 0, 5, 5, 17], dtype=np.int32)
    x = torch.empty((5, 24), dtype=torch.float32, device="cuda")
    kernels.embed(x, dev(table, DT[dtype]), dev(ids))
    assert np.array_equal(x.cpu().numpy().astype(np.float64), as_stored(table, dtype)[ids])
    out = torch.empty((3, 24), dtype=torch.float32, device="cuda")
    kernels.gather_rows(out, x, dev(np.array([4, 0, 2], dtype=np.int32)))
    assert torch.equal(out, x[[4, 0, 2]])
    bad = torch.empty((1, 24), dtype=torch.float32, device="cuda")
    kernels.embed(bad, dev(table, DT[dtype]), dev(np.array([37], dtype=np.int32)))
    assert torch.isnan(bad).all()          # an id outside the table is never looked up
    # a negative id -(s + 1) is the token that the sampler left for request slot s
    last = dev(np.array([11, 3, 29], dtype=np.int32))
    kernels.embed(x, dev(table, DT[dtype]), dev(np.array([-1, 7, -3, -2, 0], dtype=np.int32)), last)
    assert np.array_equal(x.cpu().numpy().astype(np.float64), as_stored(table, dtype)[[11, 7, 29, 3, 0]])
    kernels.embed(bad, dev(table, DT[dtype]), dev(np.array([-1], dtype=np.int32)))
    assert torch.isnan(bad).all()          # without the table of last tokens a negative id is just a bad id


@pytest.mark.parametrize("d", [2048, 200, 2052])
def test_add_rmsnorm_of_many_rows(d):
    """600 rows: widths up to 2048 take the kernel with a warp per row, wider ones the block per row."""
    from kllm_b200 import kernels
    rng = np.random.default_rng(d)
    n, eps = 600, 1e-5
    x0 = (rng.standard_normal((n, d)) * 2).astype(np.float32)
    res = rng.standard_normal((n, d)).astype(np.float32)
    gain = (1 + 0.2 * rng.standard_normal(d)).astype(np.float32)
    x, out = dev(x0), torch.empty((n, d), dtype=torch.bfloat16, device="cuda")
    kernels.add_rmsnorm(x, dev(res), out, dev(gain), eps)
    close(x, x0.astype(np.float64) + res, "float32", "residual sum")
    close(out, plain.rmsnorm(x0.astype(np.float64) + res, gain, eps), "bfloat16", "norm after the sum")
    kernels.add_rmsnorm(x, None, out, dev(gain), eps)
    close(out, plain.rmsnorm(x0.astype(np.float64) + res, gain, eps), "bfloat16", "norm alone")


@pytest.mark.parametrize("d", [2048, 4096, 200])
def test_add_rmsnorm_of_a_row_does_not_depend_on_the_number_of_rows(d):
    """The same row normalised alone, among 511 and among 512 rows: bit-equal, since the
    kernel and with it the order of the sum are chosen by the width alone."""
    from kllm_b200 import kernels
    rng = np.random.default_rng(d + 1)
    x0 = (rng.standard_normal((512, d)) * 2).astype(np.float32)
    res = rng.standard_normal((512, d)).astype(np.float32)
    gain = dev((1 + 0.2 * rng.standard_normal(d)).astype(np.float32))
    outs = []
    for n in (1, 511, 512):
        x, out = dev(x0[:n]), torch.empty((n, d), dtype=torch.bfloat16, device="cuda")
        kernels.add_rmsnorm(x, dev(res[:n]), out, gain, 1e-5)
        outs.append((x[0].clone(), out[0].clone()))
    for x_row, out_row in outs[1:]:
        assert torch.equal(x_row, outs[0][0]) and torch.equal(out_row, outs[0][1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [100, 2048 + 16, 7])
def test_add_rmsnorm(dtype, d):
    from kllm_b200 import kernels
    rng = np.random.default_rng(d)
    n, eps = 6, 3e-4
    x0 = (rng.standard_normal((n, d)) * 3).astype(np.float32)
    res = rng.standard_normal((n, d)).astype(np.float32)
    gain = (1 + 0.3 * rng.standard_normal(d)).astype(np.float32)
    res_s = as_stored(res, dtype)
    x = dev(x0)
    out = torch.empty((n, d), dtype=DT[dtype], device="cuda")
    kernels.add_rmsnorm(x, dev(res, DT[dtype]), out, dev(gain), eps)
    summed = x0.astype(np.float64) + res_s
    close(x, summed, "float32", "residual sum is float32 in both dtypes")
    close(out, plain.rmsnorm(summed, gain, eps), dtype, "norm")
    if dtype == "bfloat16":            # a float32 residual beside a bfloat16 result
        x = dev(x0)
        kernels.add_rmsnorm(x, dev(res), out, dev(gain), eps)
        close(x, x0.astype(np.float64) + res, "float32", "float32 residual, unrounded")
        close(out, plain.rmsnorm(x0.astype(np.float64) + res, gain, eps), dtype, "norm after a float32 residual")
    # no residual: x untouched
    x = dev(x0)
    kernels.add_rmsnorm(x, None, out, dev(gain), eps)
    assert np.array_equal(x.cpu().numpy(), x0)
    close(out, plain.rmsnorm(x0, gain, eps), dtype, "norm without residual")
    # chosen rows: only those are normalised, x is left alone
    rows = np.array([5, 1, 1], dtype=np.int32)
    x = dev(x0)
    out3 = torch.empty((3, d), dtype=DT[dtype], device="cuda")
    kernels.add_rmsnorm(x, dev(res, DT[dtype]), out3, dev(gain), eps, rows=dev(rows))
    assert np.array_equal(x.cpu().numpy(), x0)
    close(out3, plain.rmsnorm(summed[rows], gain, eps), dtype, "norm of chosen rows")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_mul_on_strided_halves(dtype):
    from kllm_b200 import kernels
    rng = np.random.default_rng(1)
    n, f = 5, 172
    gu = (rng.standard_normal((n, 2 * f)) * 4).astype(np.float32)
    t = dev(gu, DT[dtype])
    out = torch.empty((n, f), dtype=DT[dtype], device="cuda")
    kernels.silu_mul(out, t[:, :f], t[:, f:])
    s = as_stored(gu, dtype)
    close(out, plain.silu(s[:, :f]) * s[:, f:], dtype)
    if dtype == "bfloat16":            # float32 gate/up beside a bfloat16 result (vectorised and plain forms)
        for width in (f, f - 1):
            t32 = dev(gu)
            out = torch.empty((n, width), dtype=torch.bfloat16, device="cuda")
            kernels.silu_mul(out, t32[:, :width], t32[:, f:f + width])
            g64 = gu.astype(np.float64)
            close(out, plain.silu(g64[:, :width]) * g64[:, f:f + width], dtype, f"float32 inputs, width {width}")


def paged(k, v, page_size, n_pages, rng, dtype, lengths):
    """Scatter per-request dense k, v [len, G, hd] into caches [pages, G, page_size, hd]
    through random block tables; every slot that holds nothing is NaN."""
    G, hd = k[0].shape[1:]
    kc = np.full((n_pages, G, page_size, hd), np.nan, dtype=np.float32)
    vc = np.full_like(kc, np.nan)
    free = list(rng.permutation(n_pages))
    width = max(-(-L // page_size) for L in lengths)
    table = np.full((len(lengths), width), -1, dtype=np.int32)
    for s, L in enumerate(lengths):
        for j in range(-(-L // page_size)):
            pg = int(free.pop())
            table[s, j] = pg
            lo, hi = j * page_size, min(L, (j + 1) * page_size)
            kc[pg, :, :hi - lo] = k[s][lo:hi].transpose(1, 0, 2)
            vc[pg, :, :hi - lo] = v[s][lo:hi].transpose(1, 0, 2)
    return dev(kc, DT[dtype]), dev(vc, DT[dtype]), dev(table)


def attention_case(dtype, H, G, hd, page_size, lengths, n_new, window, seed, plant=None, kernel="generic",
                   splits=1):
    """Requests with ``lengths`` cached tokens, the last ``n_new`` of each being this
    step's queries.  Returns (got, want) for all queries.  ``kernel``: generic, decode
    (tensor cores, every token on its own, keys cut into ``splits`` ranges) or
    prefill (tensor cores, portions)."""
    from kllm_b200 import kernels
    rng = np.random.default_rng(seed)
    ks, vs, qs, pos, req, want = [], [], [], [], [], []
    for s, (L, nn) in enumerate(zip(lengths, n_new)):
        k = rng.standard_normal((L, G, hd)).astype(np.float32)
        v = rng.standard_normal((L, G, hd)).astype(np.float32)
        q = rng.standard_normal((L, H, hd)).astype(np.float32)
        if plant:
            plant(s, q, k, v)
        ks.append(k); vs.append(v)
        full = plain.attention(as_stored(q, dtype).reshape(L, H * hd), as_stored(k, dtype).reshape(L, G * hd),
                               as_stored(v, dtype).reshape(L, G * hd), H, G, hd, window=window)
        want.append(full[L - nn:])
        qs.append(q[L - nn:].reshape(nn, H * hd))
        pos.extend(range(L - nn, L)); req.extend([s] * nn)
    kc, vc, table = paged(ks, vs, page_size, sum(-(-L // page_size) for L in lengths) + 3, rng, dtype, lengths)
    q = dev(np.concatenate(qs), DT[dtype])
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(hd)
    if kernel == "generic":
        kernels.attention_generic(out, q, kc, vc, dev(np.array(pos, np.int32)), dev(np.array(req, np.int32)), table,
                                  H, G, hd, window or 0, scale)
    elif kernel == "decode":
        kernels.attention_decode(out, q, kc, vc, dev(np.array(pos, np.int32)), dev(np.array(req, np.int32)), table,
                                 H, G, hd, window or 0, scale, splits)
    elif kernel in ("dispatch", "simt"):
        # the way the attention part calls it: the kernel is chosen from the step's shape
        from types import SimpleNamespace
        ctx = SimpleNamespace(
            n_tokens=len(pos), n_requests=len(lengths), positions=dev(np.array(pos, np.int32)),
            token_req=dev(np.array(req, np.int32)), q_start=dev(np.concatenate([[0], np.cumsum(n_new)]).astype(np.int32)),
            start_pos=dev(np.array([L - nn for L, nn in zip(lengths, n_new)], dtype=np.int32)),
            host_n_new=list(n_new), all_single=all(c == 1 for c in n_new), max_ctx=max(lengths), split_bound=0)
        fn = kernels.attention if kernel == "dispatch" else kernels.attention_simt
        fn(out, q, kc, vc, ctx, table, H, G, hd, window or 0, scale)
        kernels.check_status("cuda")
    else:
        q_start = np.concatenate([[0], np.cumsum(n_new)]).astype(np.int32)
        start_pos = np.array([L - nn for L, nn in zip(lengths, n_new)], dtype=np.int32)
        fn, extra = kernels.attention_prefill, {}
        if kernel.startswith("tcgen05"):           # "tcgen05": the default form for the head size; else named
            fn = kernels.attention_prefill_tcgen05
            extra = {"probabilities": kernel.split("_")[1]} if "_" in kernel else {}
        fn(out, q, kc, vc, dev(q_start), dev(start_pos), table, len(lengths), H, G, hd, window or 0, scale, **extra)
        if kernel.startswith("tcgen05"):
            kernels.check_status("cuda")
    return out, np.concatenate(want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,hd,page", [(6, 2, 80, 8), (5, 5, 48, 16), (7, 1, 16, 3), (2, 1, 256, 32)])
def test_attention_shapes_pages_and_mixed_query_lengths(dtype, H, G, hd, page):
    lengths, n_new = [70, 1, 33, 129], [70, 1, 2, 1]      # a whole prompt, a first token, a portion, a decode
    got, want = attention_case(dtype, H, G, hd, page, lengths, n_new, None, seed=H * hd)
    assert not torch.isnan(got).any(), "a slot beyond a request's length was read"
    close(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,hd,page", [(6, 2, 80, 8), (5, 5, 48, 16), (7, 1, 16, 3), (2, 1, 256, 32), (32, 4, 64, 64),
                                         (32, 8, 128, 16), (3, 1, 36, 5)])
@pytest.mark.parametrize("window", [None, 40, 300])
def test_cuda_core_attention_portions_and_decoding_tokens(dtype, H, G, hd, page, window):
    """The float32 path's attention (register-tiled products on the CUDA cores): portions of
    any length beside single tokens, decoding tokens first as the scheduler orders them
    (contexts over 256 keys are cut into chunks and merged), all single, windows that end
    inside chunks and tiles."""
    for lengths, n_new in (([700, 257, 1, 70, 33, 129], [1, 1, 1, 70, 2, 64]),
                           ([300, 700, 1, 257, 256, 513], [1, 1, 1, 1, 1, 1]),
                           ([70, 600], [70, 333])):
        got, want = attention_case(dtype, H, G, hd, page, lengths, n_new, window, seed=H * hd + len(lengths),
                                   kernel="simt")
        assert not torch.isnan(got.float()).any(), "a slot beyond a request's length was read"
        close(got, want, dtype, f"lengths {lengths}")


@pytest.mark.parametrize("gs", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("window", [None, 300])
def test_float32_decode_attention_every_group_width(gs, hd, window):
    """Decoding tokens in float32 at head sizes 64 and 128 take a kernel of their own (every
    thread of the CTA works on a chunk of one token's keys): every width of a kv group it is
    built for, contexts that end inside a chunk, a sub-tile and a page, one kv head and
    three, beside a first token."""
    for G, page in ((1, 16), (3, 5)):
        lengths = [700, 257, 1, 300, 513, 1000, 129]
        got, want = attention_case("float32", G * gs, G, hd, page, lengths, [1] * len(lengths), window,
                                   seed=gs * hd + G, kernel="simt")
        assert not torch.isnan(got).any(), "a slot beyond a request's length was read"
        close(got, want, "float32", f"{G * gs} heads over {G} kv heads of {hd}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuda_core_attention_finds_one_far_key_among_hundreds(dtype):
    H, G, hd, L = 4, 2, 32, 700
    far = 3

    def plant(s, q, k, v):
        q[-1] *= 0.05
        k[far, 1] = 8.0 * np.sign(q[-1, 2])
        q[-1, 2] = 3.0 * np.sign(q[-1, 2])

    for n_new in (1, 90):
        got, want = attention_case(dtype, H, G, hd, 16, [L], [n_new], None, seed=7, plant=plant, kernel="simt")
        close(got, want, dtype)
        assert np.abs(want.reshape(n_new, H, hd)[-1, 2]).max() > 0.5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 5, 16, 17, 64, 255, 257])
def test_cuda_core_attention_window_edge(dtype, window):
    H, G, hd, L = 2, 1, 16, 600

    def plant(s, q, k, v):
        outside = L - 1 - window
        if s == 0 and outside >= 0:
            k[outside, 0] = 50.0 * q[-1, 0] / np.abs(q[-1, 0]).max()
            v[outside, 0] = 1e4

    for n_new in (L, 1):
        got, want = attention_case(dtype, H, G, hd, 8, [L, 40], [n_new, 3], window, seed=window, plant=plant,
                                   kernel="simt")
        close(got, want, dtype)
        assert float(got[n_new - 1].float().abs().max()) < 100.0


TC_SHAPES = [(8, 2, 64, 16), (6, 2, 80, 8), (5, 5, 48, 16), (7, 1, 16, 3), (32, 4, 128, 64), (3, 1, 32, 16),
             (16, 1, 112, 5), (4, 4, 96, 32)]


@pytest.mark.parametrize("H,G,hd,page", TC_SHAPES)
@pytest.mark.parametrize("kernel,splits", [("decode", 1), ("decode", 3), ("decode", 8), ("prefill", 1)])
def test_tensor_core_attention_shapes_pages_and_mixed_query_lengths(kernel, splits, H, G, hd, page):
    lengths, n_new = [70, 1, 33, 129, 300], [70, 1, 2, 1, 64]
    got, want = attention_case("bfloat16", H, G, hd, page, lengths, n_new, None, seed=H * hd, kernel=kernel,
                               splits=splits)
    assert not torch.isnan(got.float()).any(), "a slot beyond a request's length was read"
    close(got, want, "bfloat16")


@pytest.mark.parametrize("H,G,hd,page", [(8, 2, 64, 16), (32, 4, 64, 64), (32, 4, 128, 64), (3, 1, 64, 5), (4, 4, 128, 16),
                                         (40, 1, 64, 16)])
@pytest.mark.parametrize("where", ["smem", "tmem"])
def test_tcgen05_attention_shapes_pages_and_mixed_query_lengths(H, G, hd, page, where):
    """Both tcgen05 kernels: the probabilities through shared memory, or kept in tensor memory."""
    lengths, n_new = [70, 1, 33, 129, 300, 500], [70, 1, 2, 1, 64, 500]
    got, want = attention_case("bfloat16", H, G, hd, page, lengths, n_new, None, seed=H * hd, kernel="tcgen05_" + where)
    assert not torch.isnan(got.float()).any(), "a slot beyond a request's length was read"
    close(got, want, "bfloat16")


@pytest.mark.parametrize("H,G,hd,page", [(8, 2, 64, 16), (32, 4, 128, 64), (6, 2, 80, 8), (3, 1, 32, 5)])
@pytest.mark.parametrize("window", [None, 40])
def test_attention_of_a_mixed_step_is_cut_into_decode_and_prefill_forms(H, G, hd, page, window, monkeypatch):
    """Decoding requests first, then portions, as the scheduler orders a step: the first
    take the decode kernel, the others the prefill kernel (tcgen05 for head sizes 64 and
    128, mma.sync else); a single-token request after a portion stays with the portions."""
    from kllm_b200 import kernels
    calls = []
    for name in ("attention_decode", "attention_prefill", "attention_prefill_tcgen05"):
        real = getattr(kernels, name)
        monkeypatch.setattr(kernels, name, lambda *a, _n=name, _r=real, **k: calls.append((_n, a[1].shape[0])) or _r(*a, **k))
    lengths, n_new = [300, 1, 129, 77, 200, 31], [1, 1, 1, 77, 64, 1]
    got, want = attention_case("bfloat16", H, G, hd, page, lengths, n_new, window, seed=H + hd, kernel="dispatch")
    assert not torch.isnan(got.float()).any()
    close(got, want, "bfloat16")
    assert calls[0] == ("attention_decode", 3)
    assert calls[1][0] == ("attention_prefill_tcgen05" if hd in (64, 128) else "attention_prefill")
    # all single: the decode form alone; none single first: the prefill form alone
    calls.clear()
    got, want = attention_case("bfloat16", H, G, hd, page, [40, 300, 7], [1, 1, 1], window, seed=3, kernel="dispatch")
    close(got, want, "bfloat16")
    got, want = attention_case("bfloat16", H, G, hd, page, [40, 300, 7], [9, 1, 1], window, seed=4, kernel="dispatch")
    close(got, want, "bfloat16")
    assert [c[0] for c in calls][0] == "attention_decode" and len(calls) == 2


@pytest.mark.parametrize("kernel,splits", [("decode", 1), ("decode", 5), ("prefill", 1), ("tcgen05_smem", 1),
                                           ("tcgen05_tmem", 1)])
@pytest.mark.parametrize("window", [1, 5, 64, 65, 200])
def test_tensor_core_attention_window_edge(kernel, splits, window):
    H, G, hd, L = 4, 2, 64, 330

    def plant(s, q, k, v):
        outside = L - 1 - window
        if s == 0 and outside >= 0:
            k[outside, :] = 50.0 * q[-1, 0] / np.abs(q[-1, 0]).max()
            v[outside, :] = 1e4

    got, want = attention_case("bfloat16", H, G, hd, 16, [L, 40, 129], [L, 3, 1], window, seed=window, plant=plant,
                               kernel=kernel, splits=splits)
    close(got, want, "bfloat16")
    assert float(got[L - 1].float().abs().max()) < 100.0


@pytest.mark.parametrize("kernel,splits", [("decode", 1), ("decode", 4), ("prefill", 1), ("tcgen05_smem", 1),
                                           ("tcgen05_tmem", 1)])
def test_tensor_core_attention_finds_one_far_key(kernel, splits):
    H, G, hd, L = 4, 2, 64, 900
    far = 3

    def plant(s, q, k, v):
        q[-1] *= 0.05
        k[far, 1] = 8.0 * np.sign(q[-1, 2])
        q[-1, 2] = 3.0 * np.sign(q[-1, 2])

    got, want = attention_case("bfloat16", H, G, hd, 16, [L], [1], None, seed=7, plant=plant, kernel=kernel,
                               splits=splits)
    close(got, want, "bfloat16")
    assert np.abs(want.reshape(1, H, hd)[0, 2]).max() > 0.5


@pytest.mark.parametrize("H,G,hd,page", [(8, 2, 64, 16), (32, 4, 128, 64), (3, 1, 32, 5), (4, 4, 96, 16)])
@pytest.mark.parametrize("splits", [1, 3, 8, 12])
def test_fused_decode_attention_rotates_appends_and_merges(H, G, hd, page, splits):
    """Against the separate kernels' math: rotate q and the new k, store k and v at the
    token's slot, attend over everything.  Run twice on one counter buffer: with the
    token-to-request table, then without it (token t is request t)."""
    fused_decode_case(H, G, hd, page, splits, None)


@pytest.mark.parametrize("H,G,hd,page", [(8, 2, 64, 16), (3, 1, 32, 5), (32, 4, 128, 64)])
@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("window", [1, 5, 64, 65, 200])
def test_fused_decode_attention_with_a_window(H, G, hd, page, splits, window):
    """The same with a window: several key ranges inside the window, window edges that
    cross 64-key tiles and pages, a first range that does not start at a tile's edge.
    The pages that the window has passed are -1 in the block table, as the cache manager
    leaves them, and every cached key and value before the window is NaN: neither may be
    read."""
    fused_decode_case(H, G, hd, page, splits, window)


def fused_decode_case(H, G, hd, page, splits, window):
    from kllm_b200 import kernels
    rng = np.random.default_rng(H * hd + splits + (window or 0))
    lengths = [70, 1, 33, 129, 300]
    theta, max_pos = 1e4, 320
    j = np.arange(hd // 2, dtype=np.float64)
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * theta ** (-2.0 * j / hd)
    cos_sin = dev(np.concatenate([np.cos(ang), np.sin(ang)], 1).astype(np.float32))
    counters = torch.zeros(64, dtype=torch.int32, device="cuda")
    for rep in range(2):
        ks, vs, want, qraw, knew, vnew = [], [], [], [], [], []
        for L in lengths:
            # history keys are stored rotated already; the last position is this step's token
            k = rng.standard_normal((L, G, hd)).astype(np.float32)
            v = rng.standard_normal((L, G, hd)).astype(np.float32)
            q = rng.standard_normal((1, H, hd)).astype(np.float32)
            kq, vq, qq = as_stored(k, "bfloat16"), as_stored(v, "bfloat16"), as_stored(q, "bfloat16")
            k_last_rot = plain.round_act_bf16(plain.rope(kq[-1:].reshape(1, G * hd), [L - 1], G, hd, theta))
            q_rot = plain.round_act_bf16(plain.rope(qq.reshape(1, H * hd), [L - 1], H, hd, theta))
            k_all = np.concatenate([kq[:-1].reshape(L - 1, G * hd), k_last_rot])
            # attention of the single query over all L keys (causal mask is the loop bound)
            sc_q = np.concatenate([np.zeros((L - 1, H * hd)), q_rot])
            full = plain.attention(sc_q, k_all, vq.reshape(L, G * hd), H, G, hd, window=window,
                                   rnd_p=plain.round_act_bf16)
            want.append(full[-1:])
            hist_k = k.copy(); hist_k[-1] = np.nan          # the slot of the new token holds nothing yet
            hist_v = v.copy(); hist_v[-1] = np.nan
            if window:
                hist_k[:max(0, L - window)] = np.nan        # what the window has passed is never read
                hist_v[:max(0, L - window)] = np.nan
            ks.append(hist_k); vs.append(hist_v)
            qraw.append(q.reshape(1, H * hd)); knew.append(k[-1:].reshape(1, G * hd)); vnew.append(v[-1:].reshape(1, G * hd))
        kc, vc, table = paged(ks, vs, page, sum(-(-L // page) for L in lengths) + 3, rng, "bfloat16", lengths)
        if window:
            # pages given back at the commit before this step (cache/manager.py: commit)
            dead = torch.tensor([[j < max(0, L - window) // page for j in range(table.shape[1])] for L in lengths])
            table = torch.where(dead.cuda(), torch.full_like(table, -1), table)
        q_t, k_t, v_t = (dev(np.concatenate(a), torch.bfloat16) for a in (qraw, knew, vnew))
        out = torch.empty_like(q_t)
        pos = dev(np.array([L - 1 for L in lengths], np.int32))
        req = dev(np.arange(len(lengths), dtype=np.int32))
        kernels.attention_decode_fused(out, q_t, k_t, v_t, cos_sin, kc, vc, pos, req if rep == 0 else None, table,
                                       counters, H, G, hd, window or 0, 1.0 / math.sqrt(hd), splits)
        assert not torch.isnan(out.float()).any()
        close(out, np.concatenate(want), "bfloat16", f"attention, run {rep}")
        assert int(counters.abs().sum()) == 0, "the counters must be zero again"
        for s, L in enumerate(lengths):
            pg, slot = int(table[s, (L - 1) // page]), (L - 1) % page
            k_rot = plain.rope(as_stored(knew[s], "bfloat16"), [L - 1], G, hd, theta).reshape(G, hd)
            close(kc[pg, :, slot], k_rot, "bfloat16", "stored key")
            assert torch.equal(vc[pg, :, slot].float().cpu(), torch.from_numpy(as_stored(vnew[s], "bfloat16").reshape(G, hd)).float())


def test_tcgen05_form_follows_the_measurements():
    from kllm_b200 import kernels
    assert kernels.tcgen05_form(128, 4, 8, 2048, 1, 2048) == "tmem"
    assert kernels.tcgen05_form(64, 8, 4, 2048, 1, 2048) == "smem"        # one prompt of 2048: its longest chain rules
    assert kernels.tcgen05_form(64, 8, 4, 8192, 1, 8192) == "tmem"        # several waves of CTAs
    assert kernels.tcgen05_form(64, 8, 4, 4096, 8, 512) == "tmem"         # many short chains
    assert kernels.tcgen05_form(64, 8, 4, 700, 1, 700) == "tmem"


def test_tensor_core_attention_refusals():
    from kllm_b200 import kernels
    q = torch.zeros(1, 34 * 64, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(2, 2, 16, 64, device="cuda", dtype=torch.bfloat16)
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(kernels.KernelError, match="at most 16"):
        kernels.attention_decode(torch.empty_like(q), q, kc, kc, z, z, z.view(1, 1), 34, 2, 64, 0, 1.0, 1)
    with pytest.raises(kernels.KernelError, match="bfloat16"):
        kernels.attention_decode(torch.empty_like(q).float(), q.float(), kc.float(), kc.float(), z, z, z.view(1, 1),
                                 34, 2, 64, 0, 1.0, 1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_one_far_key_among_hundreds(dtype):
    H, G, hd, L = 4, 2, 32, 700
    far = 3

    def plant(s, q, k, v):
        q[-1] *= 0.05
        k[far, 1] = 8.0 * np.sign(q[-1, 2])              # kv head 1 serves heads 2, 3; key 3 lines up with head 2
        q[-1, 2] = 3.0 * np.sign(q[-1, 2])

    got, want = attention_case(dtype, H, G, hd, 16, [L], [1], None, seed=7, plant=plant)
    close(got, want, dtype)
    w = want.reshape(1, H, hd)
    assert np.abs(w[0, 2]).max() > 0.5                       # the far key's value dominates head 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 5, 16, 17, 64])
def test_attention_window_edge(dtype, window):
    H, G, hd, L = 2, 1, 16, 90

    def plant(s, q, k, v):
        # the key just outside the last query's window would swamp everything if it were seen
        outside = L - 1 - window
        if s == 0 and outside >= 0:
            k[outside, 0] = 50.0 * q[-1, 0] / np.abs(q[-1, 0]).max()
            v[outside, 0] = 1e4

    got, want = attention_case(dtype, H, G, hd, 8, [L, 40], [L, 3], window, seed=window, plant=plant)
    close(got, want, dtype)
    assert float(got[L - 1].float().abs().max()) < 100.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rot", [48, 16, None])
def test_rope_append(dtype, rot):
    from kllm_b200 import kernels
    rng = np.random.default_rng(3)
    H, G, hd, page, max_pos, theta = 5, 5, 48, 8, 300, 5e5
    positions = np.array([0, 1, 7, 8, 250, 299, 64], dtype=np.int32)
    req = np.array([0, 0, 0, 0, 1, 1, 2], dtype=np.int32)
    n = len(positions)
    qkv = rng.standard_normal((n, (H + 2 * G) * hd)).astype(np.float32)
    table = np.full((3, 40), -1, dtype=np.int32)
    pages = rng.permutation(60)
    for s in range(3):
        table[s] = pages[s * 20:s * 20 + 20].repeat(2)[:40] if False else np.resize(pages[s * 20:(s + 1) * 20], 40)
    table[:, 20:] = -1
    table[1, 20:38] = np.arange(100, 118)               # request 1 reaches position 299: 38 pages
    kc = torch.full((120, G, page, hd), float("nan"), dtype=DT[dtype], device="cuda")
    vc = torch.full_like(kc, float("nan"))
    t = dev(qkv, DT[dtype])
    q, k, v = t[:, :H * hd], t[:, H * hd:(H + G) * hd], t[:, (H + G) * hd:]
    cos_sin = None
    if rot:
        j = np.arange(rot // 2, dtype=np.float64)
        ang = np.arange(max_pos, dtype=np.float64)[:, None] * theta ** (-2.0 * j / rot)
        cos_sin = dev(np.concatenate([np.cos(ang), np.sin(ang)], 1).astype(np.float32))
    kernels.rope_append(q, k, v, cos_sin, dev(positions), dev(req), dev(table), kc, vc, H, G, hd)
    s = as_stored(qkv, dtype)

    def rotated(x, heads):
        x = x.reshape(n, heads, hd).copy()
        if rot:
            x[:, :, :rot] = plain.rope(x[:, :, :rot].reshape(n, heads * rot), positions, heads, rot, theta).reshape(n, heads, rot)
        return x

    close(q, rotated(s[:, :H * hd], H).reshape(n, H * hd), dtype, "q")
    kw, vw = rotated(s[:, H * hd:(H + G) * hd], G), s[:, (H + G) * hd:].reshape(n, G, hd)
    written = torch.zeros(120 * page, dtype=torch.bool)
    for i in range(n):
        pg, slot = table[req[i], positions[i] // page], positions[i] % page
        close(kc[pg, :, slot], kw[i], dtype, f"k of token {i}")
        close(vc[pg, :, slot], vw[i], dtype, f"v of token {i}")
        written[pg * page + slot] = True
    untouched = torch.isnan(kc.float()).all(dim=3).all(dim=1).reshape(-1).cpu()
    assert torch.equal(untouched, ~written), "a slot other than the tokens' own was written"


def test_rope_q_only_leaves_no_cache_write():
    from kllm_b200 import kernels
    q = torch.randn(3, 2 * 16, device="cuda")
    q0 = q.clone()
    cs = torch.cat([torch.ones(10, 8), torch.zeros(10, 8)], 1).cuda()
    kernels.rope_append(q, q, q, cs, dev(np.array([1, 2, 3], np.int32)), dev(np.zeros(3, np.int32)), None, None, None, 2, 1, 16)
    assert torch.equal(q, q0)               # cos 1, sin 0: identity


def test_sampling_greedy_first_maximum_and_temperature():
    from kllm_b200 import kernels
    rng = np.random.default_rng(5)
    V = 1000 + 3
    z = rng.standard_normal((6, V)).astype(np.float32)
    z[0, 17] = z[0, 900] = 9.0                     # a tie: the first wins
    z[1, V - 1] = 12.0                             # the last element
    z[2, :] = -1.0                                 # all equal: index 0
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    kernels.sample(out, dev(z), None, None)
    assert out.tolist()[:3] == [17, V - 1, 0]
    assert out.tolist() == [plain.argmax_first(r) for r in z]
    # temperature: the chosen index brackets u in the CDF of softmax(z / T)
    temps = np.array([0.8, 0.0, 1.5, 0.3, 1.0, 2.0], dtype=np.float32)
    for u in (0.0, 0.123, 0.5, 0.87, 0.999999):
        us = np.full(6, u, dtype=np.float32)
        kernels.sample(out, dev(z), dev(temps), dev(us))
        got = out.tolist()
        for r in range(6):
            if temps[r] <= 0:
                assert got[r] == plain.argmax_first(z[r])
                continue
            cdf = np.cumsum(plain.temperature_probs(z[r], temps[r]))
            i = got[r]
            lo = cdf[i - 1] if i else 0.0
            assert lo - 1e-5 <= u <= cdf[i] + 1e-5, (r, u, i, lo, cdf[i])
    # the choice also goes to the request slot's entry of the table that the next embedding reads
    last = torch.full((10,), -7, dtype=torch.int32, device="cuda")
    slots = dev(np.array([4, 0, 9, 2, 7, 5], dtype=np.int32))
    kernels.sample(out, dev(z), dev(temps), dev(np.full(6, 0.3, np.float32)), last, slots)
    assert last[slots.long()].tolist() == out.tolist() and last[[1, 3, 6, 8]].tolist() == [-7] * 4
    kernels.sample(out, dev(z), None, None, last, slots)
    assert last[slots.long()].tolist() == [plain.argmax_first(r) for r in z]
    with pytest.raises(kernels.KernelError, match="go together"):
        kernels.sample(out, dev(z), None, None, last, None)
    # the kernel can also leave its choices in pinned host memory by itself
    pinned = torch.full((6,), -1, dtype=torch.int32).pin_memory()
    kernels.sample(out, dev(z), None, None, host_out=pinned)
    torch.cuda.synchronize()
    assert pinned.tolist() == out.tolist() == [plain.argmax_first(r) for r in z]
    with pytest.raises(kernels.KernelError, match="pinned"):
        kernels.sample(out, dev(z), None, None, host_out=torch.zeros(6, dtype=torch.int32))
    # many draws follow the distribution
    zz = np.array([[2.0, 1.0, 0.0, -1.0, 3.0]], dtype=np.float32).repeat(4000, 0)
    us = ((np.arange(4000) + 0.5) / 4000).astype(np.float32)
    out = torch.empty(4000, dtype=torch.int32, device="cuda")
    kernels.sample(out, dev(zz), dev(np.full(4000, 0.7, np.float32)), dev(us))
    freq = np.bincount(out.cpu().numpy(), minlength=5) / 4000
    assert np.abs(freq - plain.temperature_probs(zz[0], 0.7)).max() < 2e-3


def test_linear_is_true_float32_and_bf16_accumulates_in_float32():
    from kllm_b200 import kernels
    rng = np.random.default_rng(9)
    x = rng.standard_normal((33, 1000)).astype(np.float32)
    w = rng.standard_normal((77, 1000)).astype(np.float32)
    y = kernels.linear(dev(x), dev(w))
    want = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(y.cpu().numpy() - want).max() < 2e-4          # TF32 would be off by ~3e-2 here
    yb = kernels.linear(dev(x, torch.bfloat16), dev(w, torch.bfloat16), out_dtype=torch.float32)
    wb = plain.round_bf16(x).astype(np.float64) @ plain.round_bf16(w).astype(np.float64).T
    assert yb.dtype == torch.float32 and np.abs(yb.cpu().numpy() - wb).max() < 2e-3


@pytest.mark.parametrize("n", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(48, 64), (2560, 2048), (100, 96), (2048, 5632), (33, 4096)])
def test_skinny_gemm_prologues_and_epilogues(n, N, K):
    from kllm_b200 import kernels
    rng = np.random.default_rng(n * 1000 + N)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    w2 = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    x = rng.standard_normal((n, K)).astype(np.float32)
    ws, w2s, xs = as_stored(w, "bfloat16"), as_stored(w2, "bfloat16"), as_stored(x, "bfloat16")
    wt, w2t, xt = dev(w, torch.bfloat16), dev(w2, torch.bfloat16), dev(x, torch.bfloat16)
    want = xs @ ws.T
    close(kernels.skinny_gemm(wt, x=xt, epilogue="bf16"), want, "bfloat16", "bf16 store")
    close(kernels.skinny_gemm(wt, x=xt, epilogue="f32"), want, "float32", "f32 store")
    base = rng.standard_normal((n, N)).astype(np.float32)
    acc = dev(base)
    kernels.skinny_gemm(wt, x=xt, epilogue="add", out=acc)
    close(acc, base.astype(np.float64) + want, "float32", "residual add")
    g, u = xs @ ws.T, xs @ w2s.T
    close(kernels.skinny_gemm(wt, x=xt, weight_up=w2t, epilogue="swiglu"), plain.silu(g) * u, "bfloat16", "swiglu")
    # norm prologue, on gathered rows of a larger float32 matrix
    big = (rng.standard_normal((n + 5, K)) * 2).astype(np.float32)
    gain = (1 + 0.2 * rng.standard_normal(K)).astype(np.float32)
    rows = rng.permutation(n + 5)[:n].astype(np.int32)
    xn = plain.round_act_bf16(plain.rmsnorm(big[rows], gain, 1e-5))
    got = kernels.skinny_gemm(wt, x_f32=dev(big), gain=dev(gain), eps=1e-5, rows=dev(rows), epilogue="f32")
    close(got, xn @ ws.T, "bfloat16", "norm prologue (a rounding of xn may flip)")
    got = kernels.skinny_gemm(wt, x_f32=dev(big[:n].copy()), gain=dev(gain), eps=1e-5, epilogue="bf16")
    close(got, plain.round_act_bf16(plain.rmsnorm(big[:n], gain, 1e-5)) @ ws.T, "bfloat16", "norm prologue, no gather")


@pytest.mark.parametrize("n", [1, 3, 8])
@pytest.mark.parametrize("N,K", [(48, 128), (2560, 2048), (101, 384), (2048, 5632), (33, 4096), (2, 256)])
def test_float32_skinny_gemm_prologues_and_epilogues(n, N, K):
    """The float32 path's weight-streaming product (true 32-bit FMAs on the CUDA cores)
    against float64, and bit-equal rows whatever the number of rows in the call."""
    from kllm_b200 import kernels
    rng = np.random.default_rng(n * 1000 + N + K)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    w2 = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    x = rng.standard_normal((n, K)).astype(np.float32)
    wt, w2t, xt = dev(w), dev(w2), dev(x)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    got = kernels.skinny_gemm(wt, x=xt, epilogue="store")
    assert got.dtype == torch.float32
    close(got, want, "float32", "store")
    alone = kernels.skinny_gemm(wt, x=xt[n - 1:], epilogue="f32")
    assert torch.equal(alone[0], got[n - 1]), "a row's sum must not depend on the other rows of the call"
    base = rng.standard_normal((n, N)).astype(np.float32)
    acc = dev(base)
    kernels.skinny_gemm(wt, x=xt, epilogue="add", out=acc)
    close(acc, base.astype(np.float64) + want, "float32", "residual add")
    u = x.astype(np.float64) @ w2.astype(np.float64).T
    close(kernels.skinny_gemm(wt, x=xt, weight_up=w2t, epilogue="swiglu"), plain.silu(want) * u, "float32", "swiglu")
    big = (rng.standard_normal((n + 5, K)) * 2).astype(np.float32)
    gain = (1 + 0.2 * rng.standard_normal(K)).astype(np.float32)
    rows = rng.permutation(n + 5)[:n].astype(np.int32)
    xn = plain.rmsnorm(big[rows], gain, 1e-5)
    got = kernels.skinny_gemm(wt, x_f32=dev(big), gain=dev(gain), eps=1e-5, rows=dev(rows), epilogue="f32")
    close(got, xn @ w.astype(np.float64).T, "float32", "norm prologue on gathered rows")
    got = kernels.skinny_gemm(wt, weight_up=w2t, x_f32=dev(big[:n].copy()), gain=dev(gain), eps=1e-5, epilogue="swiglu")
    xn = plain.rmsnorm(big[:n], gain, 1e-5)
    close(got, plain.silu(xn @ w.astype(np.float64).T) * (xn @ w2.astype(np.float64).T), "float32", "norm -> swiglu")


def test_float32_skinny_gemm_adds_a_long_k_in_slices():
    from kllm_b200 import kernels
    rng = np.random.default_rng(77)
    n, N, K = 5, 50, 14336
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((n, K)).astype(np.float32)
    w[:, K - 1] = 0.5
    x[:, K - 1] = 8.0
    base = rng.standard_normal((n, N)).astype(np.float32)
    acc = dev(base)
    kernels.skinny_gemm(dev(w), x=dev(x), epilogue="add", out=acc)
    close(acc, base.astype(np.float64) + x.astype(np.float64) @ w.astype(np.float64).T, "float32", "sliced residual add")


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (200, 264, 136), (77, 520, 72), (300, 96, 1000), (1000, 1544, 520)])
@pytest.mark.parametrize("bn", [0, 256, 192, 64])
def test_tcgen05_gemm_epilogues(M, N, K, bn):
    """The tensor-core product with each epilogue, at sizes with ragged edges in every
    direction (rows, columns, k) and tiles narrower than the matrix and wider."""
    from kllm_b200 import kernels
    rng = np.random.default_rng(M + N + K)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    w2 = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    ws, w2s, xs = as_stored(w, "bfloat16"), as_stored(w2, "bfloat16"), as_stored(x, "bfloat16")
    wt, w2t, xt = dev(w, torch.bfloat16), dev(w2, torch.bfloat16), dev(x, torch.bfloat16)
    want = xs @ ws.T
    close(kernels.gemm(xt, wt, epilogue="f32", bn=bn), want, "float32", "f32 store")
    close(kernels.gemm(xt, wt, epilogue="bf16", bn=bn), want, "bfloat16", "bf16 store")
    base = rng.standard_normal((M, N)).astype(np.float32)
    acc = dev(base)
    kernels.gemm(xt, wt, epilogue="add", out=acc, bn=bn)
    close(acc, base.astype(np.float64) + want, "float32", "residual add")
    got = kernels.gemm(xt, wt, weight_up=w2t, epilogue="swiglu", bn=bn)
    close(got, plain.silu(want) * (xs @ w2s.T), "bfloat16", "swiglu")
    kernels.check_status("cuda")


def test_tcgen05_gemm_rows_do_not_depend_on_the_batch():
    """A row's result is the same bits alone in a small batch and among many rows."""
    from kllm_b200 import kernels
    rng = np.random.default_rng(5)
    w = dev((rng.standard_normal((300, 200)) * 0.05).astype(np.float32), torch.bfloat16)
    x = dev(rng.standard_normal((333, 200)).astype(np.float32), torch.bfloat16)
    whole = kernels.gemm(x, w, epilogue="f32")
    part = kernels.gemm(x[130:141], w, epilogue="f32")
    assert torch.equal(whole[130:141], part)


def test_tcgen05_gemm_refusals():
    from kllm_b200 import kernels
    w = torch.zeros(64, 36, device="cuda", dtype=torch.bfloat16)
    x = torch.zeros(40, 36, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(kernels.KernelError, match="not supported"):
        kernels.gemm(x, w)                                    # k is no multiple of 8
    w = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    x = torch.zeros(40, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(kernels.KernelError, match="accumulator width"):
        kernels.gemm(x, w, bn=100)
    with pytest.raises(kernels.KernelError, match="swiglu needs"):
        kernels.gemm(x, w, epilogue="swiglu")
    with pytest.raises(kernels.KernelError, match="add"):
        kernels.gemm(x, w, epilogue="add")
    assert not kernels.gemm_fits(x.float(), w, torch.empty(40, 64, device="cuda"), "f32")
    assert kernels.gemm_pays(2048, 5632, "swiglu") and not kernels.gemm_pays(40, 96, "swiglu")


def test_skinny_gemm_refusals():
    from kllm_b200 import kernels
    w = torch.zeros(16, 40, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(kernels.KernelError, match="not supported"):
        kernels.skinny_gemm(w, x=torch.zeros(2, 40, device="cuda", dtype=torch.bfloat16))
    w = torch.zeros(16, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(kernels.KernelError, match="not supported"):
        kernels.skinny_gemm(w, x=torch.zeros(17, 64, device="cuda", dtype=torch.bfloat16))
    assert not kernels.skinny_fits(8, 64, torch.float32) and kernels.skinny_fits(16, 5632, torch.bfloat16)
    assert kernels.skinny_fits(8, 5632, torch.float32) and not kernels.skinny_fits(9, 2048, torch.float32)
    assert not kernels.skinny_fits(8, 14336, torch.float32) and kernels.skinny_fits(8, 14336, torch.float32, sliced=True)
    assert not kernels.skinny_fits(16, 14336, torch.bfloat16)
    assert kernels.skinny_fits(16, 14336, torch.bfloat16, sliced=True)
    assert not kernels.skinny_fits(16, 14336 + 8, torch.bfloat16, sliced=True)


@pytest.mark.parametrize("n,N,K", [(8, 72, 14336), (13, 40, 14336), (16, 24, 6016), (3, 50, 11200)])
def test_skinny_gemm_adds_a_long_k_in_slices(n, N, K):
    """A width too long for shared memory: the adding product takes it in column slices
    of the weight matrix (rows at a stride), and a far column still counts."""
    from kllm_b200 import kernels
    rng = np.random.default_rng(n + N + K)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((n, K)).astype(np.float32)
    w[:, K - 1] = 0.5                                   # the last column alone moves every output
    x[:, K - 1] = 8.0
    ws, xs = as_stored(w, "bfloat16"), as_stored(x, "bfloat16")
    base = rng.standard_normal((n, N)).astype(np.float32)
    acc = dev(base)
    kernels.skinny_gemm(dev(w, torch.bfloat16), x=dev(x, torch.bfloat16), epilogue="add", out=acc)
    close(acc, base.astype(np.float64) + xs @ ws.T, "float32", "sliced residual add")
    # a slice of columns given by the caller: rows at a stride, start not at the matrix's first column
    lo, hi = 64, 64 + 4096
    acc2 = dev(base)
    kernels.skinny_gemm(dev(w, torch.bfloat16)[:, lo:hi], x=dev(x, torch.bfloat16)[:, lo:hi], epilogue="add", out=acc2)
    close(acc2, base.astype(np.float64) + xs[:, lo:hi] @ ws[:, lo:hi].T, "float32", "strided weight rows")
    kernels.check_status("cuda")


def test_kernels_refuse_what_they_cannot_take():
    from kllm_b200 import kernels
    x = torch.zeros(2, 8)
    with pytest.raises(kernels.KernelError, match="CUDA"):
        kernels.add_rmsnorm(x, None, x.clone(), torch.ones(8), 1e-5)
    q = torch.zeros(1, 2 * 272, device="cuda")
    kc = torch.zeros(1, 1, 4, 272, device="cuda")
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(kernels.KernelError, match="head size"):
        kernels.attention_generic(torch.empty_like(q), q, kc, kc, z, z, z.view(1, 1), 2, 1, 272, 0, 1.0)
    with pytest.raises(kernels.KernelError, match="float32 or bfloat16"):
        kernels.silu_mul(torch.zeros(1, 4, device="cuda", dtype=torch.float16),
                         torch.zeros(1, 4, device="cuda", dtype=torch.float16),
                         torch.zeros(1, 4, device="cuda", dtype=torch.float16))
