"""Each request alone and whole: one step, logits at every position, against the
plain implementation; float32 and bfloat16; both tiny configurations."""
import numpy as np
import pytest

from helpers import assert_close, make_weights, plain_logits, prompts_for, write_model_dir

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 31, 64], "B": [1, 3, 40, 100, 128, 200]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompts(tmp_path, name, dtype):
    from kllm_b200.engine import Engine, Options, StepEntry
    cfg, w = make_weights(name, dtype)
    d = write_model_dir(str(tmp_path / name), cfg, w)
    eng = Engine(d, Options(dtype=dtype, max_seq=cfg["max_position_embeddings"], block_size=16,
                            num_blocks=32, max_batch=4))
    for ids in prompts_for(cfg, LENGTHS[name], seed=1):
        req = eng.cache.open()
        logits = eng.step([StepEntry(req, ids, list(range(len(ids))))]).cpu().numpy()
        eng.cache.close(req)
        want = plain_logits(w, cfg, ids, dtype)
        assert logits.shape == want.shape
        assert_close(logits, want, dtype, f"{name} {dtype} len {len(ids)}")
    eng.cache.audit()
    eng.close()
