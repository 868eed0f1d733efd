"""Steps of few tokens run the fused products (norm inside the product, residual add and SwiGLU behind it).
They must agree with the plain way (every norm, add and SwiGLU a kernel of its own) and with the oracle."""
import pytest
import torch

import replay_lib as rl
from helpers import TINY, TOL_BF16, make_model, plain_logits, rel_err, seeded_ids

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_fused_and_plain_steps_agree(model_root, name):
    from beglin_b200 import Engine
    cfg, _, page = TINY[name]
    folder = make_model(model_root, name, seed=11, dtype=torch.bfloat16)
    ids = seeded_ids(40, cfg["vocab_size"], 5)
    want = plain_logits(folder, ids)
    outs = {}
    for fuse in (True, False):
        eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=256, page_size=page, max_requests=2, fuse=fuse)
        rl.poison(eng)
        layer = eng.model.blocks[0]
        assert layer.mixer.qkv.fuses(4) == fuse and layer.feed_forward.down.fuses(4) == fuse
        assert not layer.mixer.qkv.fuses(17)                       # only few-token steps
        rows = [eng.step([("r", ids[:20], list(range(20)))])]      # a portion (plain way in both engines)
        for t in range(20, 40, 4):                                 # then four tokens at a time (fused when allowed)
            rows.append(eng.step([("r", ids[t:t + 4], [0, 1, 2, 3])]))
        outs[fuse] = torch.cat(rows).cpu()
        assert rel_err(outs[fuse], want) < TOL_BF16, (name, fuse)
    assert rel_err(outs[True], outs[False]) < TOL_BF16 / 2
    assert torch.equal(outs[True][:20], outs[False][:20])          # the portion ran the same kernels


def test_fused_swiglu_needs_blocks_of_64(model_root):
    from beglin_b200 import Engine
    for name, block in (("A", 64), ("B", 0)):                      # intermediate sizes 128 and 200
        folder = make_model(model_root, name, seed=3, dtype=torch.bfloat16)
        eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=128, page_size=TINY[name][2], max_requests=1)
        assert eng.model.blocks[0].feed_forward.block == block
