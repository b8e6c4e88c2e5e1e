"""GraphedFFNStack: a list of TwELLGatedMLP modules replayed as one CUDA graph."""
import pytest
import torch

from oracle import ffn_oracle as fo
from sparser_faster_llms_b200 import stack, synthetic, twell

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def test_graphed_stack_matches_eager_modules_and_dense_reference():
    L, B, d, h = 3, 8, 1024, 2048
    ffns = [synthetic.make_ffn(d, h, seed=60 + l, density=0.03, skew_sigma=1.0) for l in range(L)]
    mods = [twell.TwELLGatedMLP(500 + l, f.gate.to(DEV), f.up.to(DEV), f.down.to(DEV))
            for l, f in enumerate(ffns)]
    x = torch.stack([synthetic.make_tokens(B, d, seed=70 + l) for l in range(L)])
    runner = stack.GraphedFFNStack(mods, B)
    y1 = runner.run(x.pin_memory()).clone()
    y2 = runner.run().clone()
    assert torch.equal(y1, y2)
    for l in range(L):
        eager = mods[l](x[l].to(DEV)).cpu()
        assert torch.equal(eager, y1[l])
        ref = fo.dense_ffn(x[l], ffns[l].gate, ffns[l].up, ffns[l].down)
        _, rel = fo.max_abs_and_rel_l2(y1[l].float(), ref)
        assert rel < 1.2e-2
    last = stack.GraphedFFNStack(mods, B, return_last_only=True)
    assert torch.equal(last.run(x.pin_memory()), y1[-1])
    with pytest.raises(ValueError):
        runner.run(torch.zeros(L, B + 1, d, dtype=torch.bfloat16))
    for m in mods:
        m.destroy()
