"""The decode attention entry point that brings its own scratch memory
(``kllm_attention_decode_static``, declared in csrc/attention_tc_static.h).

It is meant for callers that cannot call cudaMalloc: code living in somebody
else's memory pool or fixed arena, or a loop that must never enter the allocator.
Here it is called the way such a caller would, through the exported C symbol of
the shared library with raw device pointers, twice in a row on different inputs
(the second call finds the first call's leftovers in the shared scratch), and each
result is held against the regular entry point's, which gets freshly allocated
scratch buffers, and against the plain float64 formula, so that a fault the two
entry points shared would show as well.  The file sorts last so that a run which stops at the first
failure has already run every other test.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1.6e-2      # of the largest |value|: the bound of the other bfloat16 kernel tests


def make_case(seed, H, G, hd, page, lengths):
    """Requests of the given cached lengths, one query token each (the last)."""
    rng = np.random.default_rng(seed)
    n_pages = sum(-(-L // page) for L in lengths) + 2
    kc = torch.full((n_pages, G, page, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    vc = torch.full_like(kc, float("nan"))
    free = list(rng.permutation(n_pages))
    width = max(-(-L // page) for L in lengths)
    table = np.full((len(lengths), width), -1, dtype=np.int32)
    for s, L in enumerate(lengths):
        k = torch.from_numpy(rng.standard_normal((L, G, hd)).astype(np.float32)).to(torch.bfloat16).cuda()
        v = torch.from_numpy(rng.standard_normal((L, G, hd)).astype(np.float32)).to(torch.bfloat16).cuda()
        for j in range(-(-L // page)):
            pg = int(free.pop())
            table[s, j] = pg
            lo, hi = j * page, min(L, (j + 1) * page)
            kc[pg, :, :hi - lo] = k[lo:hi].transpose(0, 1)
            vc[pg, :, :hi - lo] = v[lo:hi].transpose(0, 1)
    q = torch.from_numpy(rng.standard_normal((len(lengths), H * hd)).astype(np.float32)).to(torch.bfloat16).cuda()
    pos = torch.tensor([L - 1 for L in lengths], dtype=torch.int32, device="cuda")
    req = torch.arange(len(lengths), dtype=torch.int32, device="cuda")
    return q, kc, vc, pos, req, torch.from_numpy(table).cuda()


def plain_answer(q, kc, vc, table, H, G, hd, page, lengths):
    """The float64 formula (tests/plain) on the same bfloat16 values, read back through
    the block table: the last token of each request attends to all of its keys."""
    from plain import llama_plain as plain
    rows = []
    tab = table.cpu().numpy()
    for s, L in enumerate(lengths):
        pages = tab[s, :-(-L // page)]
        k = kc[pages].float().cpu().numpy().transpose(0, 2, 1, 3).reshape(-1, G * hd)[:L]
        v = vc[pages].float().cpu().numpy().transpose(0, 2, 1, 3).reshape(-1, G * hd)[:L]
        qs = np.zeros((L, H * hd))
        qs[-1] = q[s].float().cpu().numpy()
        rows.append(plain.attention(qs, k, v, H, G, hd)[-1])
    return np.stack(rows)


def call_static(lib, out, q, kc, vc, pos, req, table, H, G, hd, splits, window=0):
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    fn = lib.kllm_attention_decode_static
    fn.restype = ctypes.c_int
    return fn(p(out), p(q), ctypes.c_int64(q.stride(0)), p(kc), p(vc), p(pos), p(req), p(table),
              ctypes.c_int(table.shape[1]), ctypes.c_int(q.shape[0]), ctypes.c_int(H), ctypes.c_int(G),
              ctypes.c_int(hd), ctypes.c_int(kc.shape[2]), ctypes.c_int(window),
              ctypes.c_float(1.0 / math.sqrt(hd)), ctypes.c_int(splits),
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_entry_point_matches_the_regular_one_twice_in_a_row():
    from kllm_b200 import kernels
    from kllm_b200.csrc.build import load_library
    H, G, hd, page = 8, 2, 64, 16
    lib = load_library("attention_tc", {"KLLM_HD": hd})
    for seed, lengths, splits in ((1, [300, 17, 129, 64], 4), (2, [70, 511, 1], 7)):
        q, kc, vc, pos, req, table = make_case(seed, H, G, hd, page, lengths)
        want = torch.empty_like(q)
        kernels.attention_decode(want, q, kc, vc, pos, req, table, H, G, hd, 0, 1.0 / math.sqrt(hd), splits)
        got = torch.full_like(q, float("nan"))
        rc = call_static(lib, got, q, kc, vc, pos, req, table, H, G, hd, splits)
        if rc != 0:
            lib.kllm_last_error_attention_tc.restype = ctypes.c_char_p
            pytest.fail(f"kllm_attention_decode_static returned {rc}: {lib.kllm_last_error_attention_tc().decode()}")
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        scale = float(want.float().abs().max())
        assert float((got.float() - want.float()).abs().max()) <= TOL * scale
        formula = plain_answer(q, kc, vc, table, H, G, hd, page, lengths)
        assert float(np.abs(got.float().cpu().numpy() - formula).max()) <= TOL * float(np.abs(formula).max())


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from kllm_b200.csrc.build import load_library
    H, G, hd, page = 8, 2, 64, 16
    lib = load_library("attention_tc", {"KLLM_HD": hd})
    q, kc, vc, pos, req, table = make_case(3, H, G, hd, page, [40] * 4)
    # 4 tokens x 8 heads x 32 splits x 66 floats fit; pretend to a batch that cannot
    big_q = q.repeat(1024, 1)
    big_pos, big_req = pos.repeat(1024), torch.zeros(4096, dtype=torch.int32, device="cuda")
    out = torch.empty_like(big_q)
    rc = call_static(lib, out, big_q, kc, vc, big_pos, big_req, table, H, G, hd, 32)
    assert rc < 0
    lib.kllm_last_error_attention_tc.restype = ctypes.c_char_p
    msg = lib.kllm_last_error_attention_tc().decode()
    assert "floats of scratch" in msg and "holds" in msg
    # one split needs no scratch at all and is always accepted
    assert call_static(lib, out, big_q, kc, vc, big_pos, big_req, table, H, G, hd, 1) == 0
    torch.cuda.synchronize()
