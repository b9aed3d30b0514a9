"""Child process of test_gpu_reference_anchor.py: the reference's own CUDA backend
(baseline/_ref/libkllm_backend.so, built from its unmodified sources) run on given
weights and prompts through its C ABI.  The backend holds one model per process, so
each configuration gets a process of its own.

    python reference_backend_child.py IN.npz OUT.npz

IN.npz: ``config`` (JSON text), ``prompts`` (JSON text, list of id lists), ``cut``
(where each prompt is cut for the second run) and the weights under their tensor
names.  OUT.npz, for prompt i:
  whole_i   logits of the last token when the prompt runs as one span
  tap_i_j   debug tap j of that run (embedding output, residual stream after every
            layer, final norm's output; backend/shim.h:128-136), [tokens, hidden]
  spans_i   logits at positions cut-1 .. n-1: the first ``cut`` tokens as one span,
            the rest one token a call, the first prompt running beside it as a second
            sequence of the batch (mixed spans through te_forward_batch)
"""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline"))
import reference_arm as ra   # noqa: E402


def main():
    src = np.load(sys.argv[1])
    cfg = json.loads(str(src["config"]))
    prompts = json.loads(str(src["prompts"]))
    cuts = [int(c) for c in src["cut"]]
    weights = {k: src[k] for k in src.files if k not in ("config", "prompts", "cut")}
    max_seq = cfg["max_position_embeddings"]
    ref = ra.Reference(cfg, max_seqs=2, max_seq=max_seq, block=16, weights=weights)
    hidden = cfg["hidden_size"]
    out = {}
    tables = ref.tables(2)
    for i, ids in enumerate(prompts):
        n = len(ids)
        ref.debug(True)
        out[f"whole_{i}"] = ref.forward(ids, [n], [0], tables[:1])[0]
        for j, tap in enumerate(ref.taps()):
            out[f"tap_{i}_{j}"] = tap.reshape(n, hidden)
        ref.debug(False)
        cut = cuts[i]
        rows = [ref.forward(ids[:cut], [cut], [0], tables[:1])[0]]
        other = prompts[0]
        fed = 0
        for t in range(cut, n):
            # the other sequence advances by a span of two tokens beside the single token
            if fed + 2 <= len(other) and fed + 2 <= max_seq:
                both = ref.forward([ids[t]] + other[fed:fed + 2], [1, 2], [t, fed], tables)
                fed += 2
            else:
                both = ref.forward([ids[t]], [1], [t], tables[:1])
            rows.append(both[0])
        out[f"spans_{i}"] = np.stack(rows)
    np.savez(sys.argv[2], **out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
