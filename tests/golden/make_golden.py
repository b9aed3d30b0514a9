"""Makes ``reference_numpy_forward.npz``: outputs of the reference project's own
numpy forward pass on a micro Llama, for ``tests/test_plain.py`` to hold the plain
implementation against.

The reference (Kartikeya-trivedi/KLLM) has no Python model code for the dense
Llama path, but ``tools/gen_reference_numpy_moe.py`` holds a numpy decoder
(``TinyMoE.forward`` :85-131 with ``rmsnorm`` :28-30, ``rope`` :33-45, ``silu``
:48-49) whose only non-Llama piece is the feed-forward ``moe()`` (:70-83).  This
script imports that module unchanged from a checkout of the reference, overrides
``moe()`` alone with the dense SwiGLU of ``backend/model.cu:1112-1115``, and runs
it on the CPU.  Everything else (norm, rotary embedding, attention with its mask
and softmax, residual order, final norm, last-row logits) is the reference's code.

    python tests/golden/make_golden.py --reference /path/to/KLLM

The weights of the micro model are written into the .npz too, so the test needs
neither the reference nor this script.
"""
import argparse
import json
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 32, "intermediate_size": 44, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 8,
    "vocab_size": 48, "max_position_embeddings": 64, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "tie_word_embeddings": False,
    # keys that TinyMoE's constructor reads and the dense path never uses
    "num_local_experts": 1, "num_experts_per_tok": 1,
}
PROMPTS = [[1, 17, 42, 10, 7], [3, 3, 3, 40, 41, 42, 43, 44, 45, 46, 47, 0, 9, 21, 30, 5, 6]]


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--reference", required=True, help="checkout of Kartikeya-trivedi/KLLM")
    ap.add_argument("--out", default=str(HERE / "reference_numpy_forward.npz"))
    args = ap.parse_args()

    sys.path.insert(0, str(Path(args.reference) / "tools"))
    import gen_reference_numpy_moe as ref  # the reference's module, unchanged
    from make_test_model import save_safetensors  # the reference's writer
    from plain.llama_plain import random_weights

    class DenseLlama(ref.TinyMoE):
        def moe(self, l, x):
            pre = f"model.layers.{l}.mlp"
            g = ref.silu(x @ self.w[f"{pre}.gate_proj.weight"].T)
            u = x @ self.w[f"{pre}.up_proj.weight"].T
            return ((g * u) @ self.w[f"{pre}.down_proj.weight"].T).astype(np.float32)

    weights = random_weights(CONFIG, seed=11, gain_std=0.1)
    out = {"config_json": np.frombuffer(json.dumps(CONFIG).encode(), dtype=np.uint8)}
    for name, arr in weights.items():
        out["w/" + name] = arr
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        (tmp / "config.json").write_text(json.dumps(CONFIG))
        save_safetensors(tmp / "model.safetensors", weights)
        for i, ids in enumerate(PROMPTS):
            m = DenseLlama(tmp)
            logits, hidden = m.forward(ids, 0, collect_hidden=True)
            out[f"p{i}/ids"] = np.asarray(ids, dtype=np.int32)
            out[f"p{i}/last_logits"] = logits
            for j, h in enumerate(hidden):
                out[f"p{i}/hidden_{j}"] = h
            # the same prompt in two portions through the reference's own cache
            m2 = DenseLlama(tmp)
            cut = max(1, len(ids) // 2)
            m2.forward(ids[:cut], 0)
            logits2, _ = m2.forward(ids[cut:], cut)
            out[f"p{i}/last_logits_two_portions"] = logits2
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, "with", len(out), "arrays")


if __name__ == "__main__":
    main()
