"""End-to-end decode loop on the GPU: the TwELL FFN variant against the dense cuBLAS variant
on the same weights, and CUDA-graph replay against eager stepping."""
import pytest
import torch

from sparser_faster_llms_b200 import decode_model as dm

pytestmark = pytest.mark.gpu


def cfg():
    return dm.DecoderConfig(layers=3, d_model=512, heads=4, head_dim=128, d_ff=2048, vocab=640,
                            max_seq=64, density=0.03, skew_sigma=1.0)


def prompt(b, s, vocab):
    return torch.randint(0, vocab, (b, s), generator=torch.Generator().manual_seed(4)).cuda()


@pytest.mark.parametrize("batch", [1, 8])
def test_twell_decoder_tracks_dense_decoder(batch):
    c = cfg()
    ids = prompt(batch, 24, c.vocab)
    sparse = dm.SparseDecoder(c, batch, ffn="twell", seed=5)
    dense = dm.SparseDecoder(c, batch, ffn="dense", seed=5)
    sparse.prefill(ids)
    dense.prefill(ids)
    # logits after the prompt: same function, bf16 rounding differs (sparse path: bf16 products)
    ref = dense.last_logits
    assert (sparse.last_logits - ref).norm() / ref.norm() < 3e-2
    # one decode step fed the same token
    sparse.ids.copy_(dense.ids)
    sparse.generate(1, use_graph=False)
    dense.generate(1, use_graph=False)
    ref = dense.last_logits
    assert (sparse.last_logits - ref).norm() / ref.norm() < 3e-2
    sparse.destroy()


def test_graph_replay_generates_the_same_tokens_as_eager_steps():
    c = cfg()
    ids = prompt(4, 16, c.vocab)
    a = dm.SparseDecoder(c, 4, ffn="twell", seed=6)
    a.prefill(ids)
    eager = a.generate(12, use_graph=False).clone()
    a.prefill(ids)
    a.capture()
    replayed = a.generate(12).clone()
    assert torch.equal(eager, replayed)
    assert int(a.pos) == 16 + 12
    a.destroy()


def test_flash_kvcache_decode_step_matches_the_sdpa_step():
    """The decode step through flash-attn's kv-cache kernel (rotary + append + attention in one
    launch) against the torch SDPA step on the same weights, where the kernel runs."""
    c = cfg()
    ids = prompt(2, 20, c.vocab)
    fast = dm.SparseDecoder(c, 2, ffn="dense", seed=7)
    if fast.attn != "flash":
        pytest.skip("flash_attn_with_kvcache does not run on this device")
    slow = dm.SparseDecoder(c, 2, ffn="dense", seed=7, attn="sdpa")
    fast.prefill(ids)
    slow.prefill(ids)
    for _ in range(3):
        fast.ids.copy_(slow.ids)  # same token into both
        fast.generate(1, use_graph=False)
        slow.generate(1, use_graph=False)
        ref = slow.last_logits
        assert (fast.last_logits - ref).norm() / ref.norm() < 2e-2
    assert int(fast.seqlens[0]) == 23 and int(fast.pos) == 23
