"""Decode loop logic on CPU with the dense FFN variant (the TwELL variant needs CUDA): the
KV-cache step must reproduce what a full forward over the longer sequence computes."""
import torch

from sparser_faster_llms_b200 import decode_model as dm


def small_cfg():
    return dm.DecoderConfig(layers=2, d_model=64, heads=4, head_dim=16, d_ff=256, vocab=97,
                            max_seq=32, density=0.2, skew_sigma=0.0)


def test_cached_decode_equals_recomputed_prefill():
    cfg = small_cfg()
    b, s, steps = 3, 9, 5
    ids = torch.randint(0, cfg.vocab, (b, s), generator=torch.Generator().manual_seed(1))
    model = dm.SparseDecoder(cfg, b, ffn="dense", seed=3, device="cpu")
    model.prefill(ids)
    toks = model.generate(steps, use_graph=False).clone()      # [steps + 1, B]
    assert toks.shape == (steps + 1, b)
    logits_cached = model.last_logits.clone()
    # the same sequence recomputed from scratch: prompt + all but the last generated token
    full = torch.cat([ids, toks[:steps].T], dim=1)
    fresh = dm.SparseDecoder(cfg, b, ffn="dense", seed=3, device="cpu")
    fresh.prefill(full)
    assert torch.equal(fresh.ids, toks[steps])
    ref = fresh.last_logits
    assert (logits_cached - ref).abs().max() <= 2e-2 * ref.abs().max()
    assert int(model.pos) == s + steps and model.host_pos == s + steps


def test_generation_is_bounded_by_max_seq():
    cfg = small_cfg()
    model = dm.SparseDecoder(cfg, 1, ffn="dense", seed=0, device="cpu")
    model.prefill(torch.zeros(1, 20, dtype=torch.long))
    try:
        model.generate(20, use_graph=False)
    except ValueError:
        return
    raise AssertionError("generation past max_seq must be refused")
