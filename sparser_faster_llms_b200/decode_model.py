"""A random-init sparse decoder around the FFN modules, for end-to-end decode ms/token.

The reference has no decode loop (``use_cache`` is forced off and its kernels need token
counts that are multiples of 256, benchmark_inference.py:147,171-177), so this module supplies
one: a Llama-style decoder (RMSNorm, rotary attention with a static KV cache, gated FFN with
ReLU, untied LM head) whose FFN is either the TwELL module of this package or the dense
bf16 formula through cuBLAS - the same weights, the same function
(``SparseMLP._forward_mlp_inference_logic``, custom_models/sparse_models.py:343-351, with the
gate shift of :mod:`synthetic` as an explicit gate bias).  Attention, norms and the LM head
are library code (cuBLAS, torch's fused RMSNorm, and for the decode step flash-attn's
``flash_attn_with_kvcache`` - rotary embedding, cache append and attention in one kernel -
where it runs on the device; torch SDPA otherwise), and in the decode step every "residual
add, then RMSNorm" pair around the FFN is one launch of this package's
``b200_residual_rmsnorm``: they are outside the sparse-FFN path and identical in both
variants.  One decode step (all layers, greedy sampling, KV-cache update, position
increment) is captured in a CUDA graph and replayed; nothing returns to the host between
tokens.

``python -m sparser_faster_llms_b200.decode_model [--batch 1,8,32] [--prompt 512]
[--generate 256]`` prints one JSON line per batch size with ms/token for both variants.
"""
from __future__ import annotations

import argparse
import json
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from . import norm, synthetic, twell


@dataclass
class DecoderConfig:
    layers: int = 28
    d_model: int = 2048
    heads: int = 16
    head_dim: int = 128
    d_ff: int = 8192
    vocab: int = 32000
    max_seq: int = 768
    rope_theta: float = 10000.0
    density: float = 0.02
    skew_sigma: float = 1.0
    eps: float = 1e-5


class DenseGatedFFN(nn.Module):
    """``(relu(x Wg^T + b) * (x Wu^T)) Wd`` through cuBLAS; weights in the TwELL layout [H, D]."""

    def __init__(self, gate, up, down, bias):
        super().__init__()
        self.register_buffer("GATE", gate)
        self.register_buffer("UP", up)
        self.register_buffer("DOWN_T", down.t().contiguous())  # [D, H] = down_proj.weight
        self.register_buffer("bias", bias.to(gate.dtype))

    def forward(self, x):
        return F.linear(torch.relu(F.linear(x, self.GATE, self.bias)) * F.linear(x, self.UP),
                        self.DOWN_T)


def _rms_norm(x, w, eps):
    return F.rms_norm(x, (x.shape[-1],), w, eps)


class SparseDecoder(nn.Module):
    """``ffn`` = "twell" (this package's sparse path) or "dense" (cuBLAS)."""

    def __init__(self, cfg: DecoderConfig, batch: int, *, ffn: str = "twell", seed: int = 0,
                 device="cuda", shard: dict | None = None, attn: str = "auto"):
        """``shard = {"rank", "world", "peer_allreduce", "fused_allreduce"}`` splits the d_ff of
        every TwELL FFN over the ranks of a process group (attention, norms and the LM head stay
        replicated); every rank then holds the same activations and generates the same tokens."""
        super().__init__()
        if ffn not in ("twell", "dense"):
            raise ValueError("ffn must be 'twell' or 'dense'")
        if attn not in ("auto", "flash", "sdpa"):
            raise ValueError("attn must be 'auto', 'flash' or 'sdpa'")
        self.cfg, self.batch, self.kind = cfg, int(batch), ffn
        self.shard = shard if (shard and shard.get("world", 1) > 1 and ffn == "twell") else None
        dev = torch.device(device)
        gen = torch.Generator().manual_seed(seed)
        bf = torch.bfloat16
        d, hd, nh = cfg.d_model, cfg.head_dim, cfg.heads

        dgen = torch.Generator(device=dev).manual_seed(seed) if dev.type == "cuda" else None

        def w(*shape):
            if dgen is not None:  # drawn on the device: a model-sized stack builds in a second
                return (torch.randn(*shape, generator=dgen, device=dev) * 0.02).to(bf)
            return (torch.randn(*shape, generator=gen) * 0.02).to(bf).to(dev)

        self.embed = w(cfg.vocab, d)
        self.lm_head = w(cfg.vocab, d)
        self.final_norm = torch.ones(d, dtype=bf, device=dev)
        self.norm1 = [torch.ones(d, dtype=bf, device=dev) for _ in range(cfg.layers)]
        self.norm2 = [torch.ones(d, dtype=bf, device=dev) for _ in range(cfg.layers)]
        self.wqkv = [w(3 * nh * hd, d) for _ in range(cfg.layers)]
        self.wo = [w(d, nh * hd) for _ in range(cfg.layers)]
        self.ffns = nn.ModuleList()
        for l in range(cfg.layers):
            f = synthetic.make_ffn(d, cfg.d_ff, seed=seed * 1000 + l, density=cfg.density,
                                   skew_sigma=cfg.skew_sigma, fold_bias=False, device=dev,
                                   generate_on_device=True)
            if self.shard is not None:
                from . import sharded
                r, w = self.shard["rank"], self.shard["world"]
                h0, h1 = sharded.shard_range(cfg.d_ff, r, w)
                gs, us, ds = (t[h0:h1].contiguous().to(dev) for t in (f.gate, f.up, f.down))
                m = sharded.ShardedTwELLGatedMLP(
                    7000 + l, gs, us, ds, rank=r, world_size=w, presharded=True,
                    peer_allreduce=self.shard.get("peer_allreduce"),
                    fused_allreduce=self.shard.get("fused_allreduce"),
                    preallocate_shared_hidden_state=True)
                m.local.set_gate_bias(f.gate_bias[h0:h1].to(dev))
                self.ffns.append(m)
                continue
            g, u, dn, b = f.gate.to(dev), f.up.to(dev), f.down.to(dev), f.gate_bias.to(dev)
            if ffn == "twell":
                m = twell.TwELLGatedMLP(7000 + l, g, u, dn, preallocate_shared_hidden_state=True)
                m.set_gate_bias(b)
            else:
                m = DenseGatedFFN(g, u, dn, b)
            self.ffns.append(m)
        # static KV cache [layers, B, S, heads, head_dim] and rotary tables
        self.k_cache = torch.zeros(cfg.layers, batch, cfg.max_seq, nh, hd, dtype=bf, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
        ang = torch.outer(torch.arange(cfg.max_seq, dtype=torch.float32), inv)
        self.cos = torch.cat([ang.cos(), ang.cos()], -1).to(dev)  # [max_seq, hd] fp32
        self.sin = torch.cat([ang.sin(), ang.sin()], -1).to(dev)
        self.cos_half = ang.cos().to(bf).to(dev)                   # [max_seq, hd / 2], decode kernel
        self.sin_half = ang.sin().to(bf).to(dev)
        self.seqlens = torch.zeros(batch, dtype=torch.int32, device=dev)  # tokens in the cache
        self.attn = self._pick_attention(attn, dev)
        self.fused_norm = dev.type == "cuda"  # residual add + RMSNorm as one library kernel
        # decode-step state (device resident; the captured graph updates it in place)
        self.ids = torch.zeros(batch, dtype=torch.long, device=dev)
        self.pos = torch.zeros(1, dtype=torch.long, device=dev)
        self.step = torch.zeros(1, dtype=torch.long, device=dev)  # row of `generated` last written
        self.arange = torch.arange(cfg.max_seq, device=dev)
        self.generated = torch.zeros(cfg.max_seq, batch, dtype=torch.long, device=dev)
        self.last_logits = torch.zeros(batch, cfg.vocab, dtype=torch.float32, device=dev)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.host_pos, self.host_step = 0, 0
        self.dev = dev

    # -- building blocks --------------------------------------------------------
    def _pick_attention(self, attn: str, dev: torch.device) -> str:
        """"flash" when flash-attn's kv-cache kernel runs on this device (probed once with a
        tiny call), else "sdpa"."""
        if attn == "sdpa" or dev.type != "cuda":
            if attn == "flash":
                raise RuntimeError("attn='flash' needs a CUDA device")
            return "sdpa"
        try:
            from flash_attn import flash_attn_with_kvcache
            q = torch.zeros(1, 1, 2, self.cfg.head_dim, dtype=torch.bfloat16, device=dev)
            kc = torch.zeros(1, 16, 2, self.cfg.head_dim, dtype=torch.bfloat16, device=dev)
            flash_attn_with_kvcache(q, kc, kc.clone(), k=q, v=q,
                                    rotary_cos=self.cos_half[:16], rotary_sin=self.sin_half[:16],
                                    cache_seqlens=torch.zeros(1, dtype=torch.int32, device=dev),
                                    causal=True, rotary_interleaved=False)
            torch.cuda.synchronize(dev)
            return "flash"
        except Exception:
            if attn == "flash":
                raise
            return "sdpa"

    def _rope(self, t, cos, sin):  # t [..., S, heads, hd]; cos/sin [S, 1, hd]
        half = t.shape[-1] // 2
        rot = torch.cat([-t[..., half:], t[..., :half]], -1)
        return (t.float() * cos + rot.float() * sin).to(t.dtype)

    def _ffn(self, l, x):  # x [B, S, D]
        b, s, d = x.shape
        return self.ffns[l](x.reshape(b * s, d)).view(b, s, d)

    def _attention(self, l, h, cos, sin, write_pos, mask, causal):
        """Attention block on the normalised hidden state ``h [B, S, D]`` -> ``[B, S, D]``."""
        cfg = self.cfg
        b, s, _ = h.shape
        nh, hd = cfg.heads, cfg.head_dim
        qkv = F.linear(h, self.wqkv[l]).view(b, s, 3, nh, hd)
        if not causal and self.attn == "flash":
            # decode step: rotary embedding of q and k, cache append at seqlens, attention
            from flash_attn import flash_attn_with_kvcache
            a = flash_attn_with_kvcache(
                qkv[:, :, 0], self.k_cache[l], self.v_cache[l], k=qkv[:, :, 1], v=qkv[:, :, 2],
                rotary_cos=self.cos_half, rotary_sin=self.sin_half, cache_seqlens=self.seqlens,
                causal=True, rotary_interleaved=False)
        else:
            qk = self._rope(qkv[:, :, :2].transpose(0, 2), cos, sin)  # [2, s, b, nh, hd] rotated
            q, k, v = qk[0].transpose(0, 1), qk[1].transpose(0, 1), qkv[:, :, 2]  # [b, s, nh, hd]
            self.k_cache[l].index_copy_(1, write_pos, k)
            self.v_cache[l].index_copy_(1, write_pos, v)
            if causal:   # prefill: attend inside the prompt only
                a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2),
                                                   v.transpose(1, 2), is_causal=True)
            else:        # decode: one query over the whole static cache, masked past `pos`
                a = F.scaled_dot_product_attention(q.transpose(1, 2),
                                                   self.k_cache[l].transpose(1, 2),
                                                   self.v_cache[l].transpose(1, 2),
                                                   attn_mask=mask)
            a = a.transpose(1, 2)
        return F.linear(a.reshape(b, s, nh * hd), self.wo[l])

    def _layer(self, l, x, cos, sin, write_pos, mask, causal):
        cfg = self.cfg
        x = x + self._attention(l, _rms_norm(x, self.norm1[l], cfg.eps), cos, sin, write_pos,
                                mask, causal)
        return x + self._ffn(l, _rms_norm(x, self.norm2[l], cfg.eps))

    def _add_norm(self, x, delta, w):
        """``(x + delta, rmsnorm(x + delta) * w)``: one library kernel on the GPU."""
        if x.is_cuda and self.fused_norm:
            return norm.residual_rmsnorm(x, delta, w, self.cfg.eps, inplace=True)
        if delta is not None:
            x = x + delta
        return x, _rms_norm(x, w, self.cfg.eps)

    # -- prefill / decode ---------------------------------------------------------
    @torch.no_grad()
    def prefill(self, prompt_ids: torch.Tensor) -> None:
        """Runs the prompt ``[B, S]``, fills the KV cache, leaves the first generated token in
        ``self.ids`` and ``S`` in ``self.pos``."""
        b, s = prompt_ids.shape
        if b != self.batch or s >= self.cfg.max_seq:
            raise ValueError("prompt does not fit this decoder's batch / max_seq")
        x = self.embed[prompt_ids]
        wp = self.arange[:s]
        cos, sin = self.cos[:s].view(s, 1, 1, -1), self.sin[:s].view(s, 1, 1, -1)
        for l in range(self.cfg.layers):
            x = self._layer(l, x, cos, sin, wp, None, True)
        logits = F.linear(_rms_norm(x[:, -1], self.final_norm, self.cfg.eps), self.lm_head).float()
        self.last_logits.copy_(logits)
        self.ids.copy_(logits.argmax(-1))
        self.pos.fill_(s)
        self.seqlens.fill_(s)
        self.step.zero_()
        self.host_pos, self.host_step = s, 0
        self.generated[0].copy_(self.ids)

    @torch.no_grad()
    def _decode_body(self) -> None:
        pos = self.pos
        x = self.embed[self.ids].unsqueeze(1)                                   # [B, 1, D]
        cos = sin = mask = None
        if self.attn != "flash":
            cos = self.cos.index_select(0, pos).view(1, 1, 1, -1)
            sin = self.sin.index_select(0, pos).view(1, 1, 1, -1)
            mask = torch.zeros(1, 1, 1, self.cfg.max_seq, dtype=x.dtype, device=self.dev)
            mask.masked_fill_((self.arange > pos).view(1, 1, 1, -1), float("-inf"))
        # residual stream x and the sub-block output not yet added to it (delta): every
        # "add, then normalise" pair is one kernel
        delta = None
        for l in range(self.cfg.layers):
            x, h = self._add_norm(x, delta, self.norm1[l])
            x, h = self._add_norm(x, self._attention(l, h, cos, sin, pos, mask, False),
                                  self.norm2[l])
            delta = self._ffn(l, h)
        x, h = self._add_norm(x, delta, self.final_norm)
        logits = F.linear(h[:, 0], self.lm_head).float()
        self.last_logits.copy_(logits)
        self.ids.copy_(logits.argmax(-1))
        self.pos.add_(1)
        self.seqlens.add_(1)
        self.step.add_(1)
        self.generated.index_copy_(0, self.step, self.ids.unsqueeze(0))

    def capture(self) -> None:
        """Captures one decode step; call after :meth:`prefill`.  The two warm-up steps that
        precede the capture are undone (position and token restored; the cache rows they wrote
        are overwritten by the replays)."""
        ids0, pos0, step0 = self.ids.clone(), self.pos.clone(), self.step.clone()
        len0 = self.seqlens.clone()
        s = torch.cuda.Stream(self.dev)
        s.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(s):
            for _ in range(2):
                self._decode_body()
        torch.cuda.current_stream(self.dev).wait_stream(s)
        torch.cuda.synchronize(self.dev)
        g = torch.cuda.CUDAGraph()
        # same stream as the warm-up: the contraction's per-stream workspace exists for it
        with torch.cuda.graph(g, stream=s):
            self._decode_body()
        self.ids.copy_(ids0)
        self.pos.copy_(pos0)
        self.step.copy_(step0)
        self.seqlens.copy_(len0)
        self.graph = g

    @torch.no_grad()
    def generate(self, steps: int, *, use_graph: bool = True) -> torch.Tensor:
        """``steps`` more greedy tokens; returns all tokens generated since the prefill,
        ``[n + 1, B]`` (row 0 is the token the prefill produced).  No host synchronisation
        between steps; ``host_pos`` tracks the position on the host."""
        if self.host_pos + steps >= self.cfg.max_seq:
            raise ValueError("generation would run past max_seq")
        if use_graph and self.graph is None:
            self.capture()
        for _ in range(steps):
            if use_graph:
                self.graph.replay()
            else:
                self._decode_body()
        self.host_pos += steps
        self.host_step += steps
        return self.generated[: self.host_step + 1]

    def destroy(self) -> None:
        for m in self.ffns:
            if hasattr(m, "destroy"):
                m.destroy()


def time_decode(cfg: DecoderConfig, batch: int, prompt: int, generate: int, ffn: str,
                seed: int = 0, reps: int = 3, shard: dict | None = None) -> dict:
    """Prefill ``prompt`` random ids, then time ``generate`` graph-replayed decode steps with
    CUDA events on the current stream; ``reps`` times from the same prompt, best and median.
    With ``shard`` (several ranks) every run starts behind a barrier and the time is the
    maximum over ranks."""
    import torch.distributed as dist
    dev = torch.device("cuda", torch.cuda.current_device())
    model = SparseDecoder(cfg, batch, ffn=ffn, seed=seed, device=dev, shard=shard)
    multi = model.shard is not None
    ids = torch.randint(0, cfg.vocab, (batch, prompt), generator=torch.Generator().manual_seed(7))
    ids = ids.to(dev)
    runs = []
    for _ in range(reps):
        if multi:
            torch.cuda.synchronize(dev)
            dist.barrier()
        model.prefill(ids)
        if model.graph is None:
            model.capture()
        model.generate(8)                      # warm-up replays
        torch.cuda.synchronize(dev)
        if multi:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        toks = model.generate(generate - 8)
        e1.record()
        torch.cuda.synchronize(dev)
        ms_run = e0.elapsed_time(e1) / (generate - 8)
        if multi:
            t = torch.tensor([ms_run], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_run = float(t.item())
        runs.append(ms_run)
    ms = min(runs)
    out = {"ffn": ffn, "ms_per_token": ms, "ms_per_token_median": sorted(runs)[len(runs) // 2],
           "tokens_per_s": batch / (ms * 1e-3),
           "first_tokens": toks[:4, 0].tolist(), "logits_checksum": float(model.last_logits.abs().sum())}
    slab = twell._SHARED_PACKED_HIDDEN_STATE
    if ffn == "twell" and slab is not None and slab.shape[0] == batch:
        # gate positives per token in the last layer of the last step (the slab all layers share)
        counts = slab.view(torch.int32)[:, ::32].long()
        out["last_layer_nnz_per_token"] = counts.sum().item() / batch
        out["last_layer_active_union"] = int(
            (twell.packed_to_dense(slab, cfg.d_ff) != 0).any(0).sum())
    model.destroy()
    del model
    torch.cuda.empty_cache()
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", default="1,8,32")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--generate", type=int, default=256)
    ap.add_argument("--layers", type=int, default=28)
    args = ap.parse_args()
    import os
    import sys
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = DecoderConfig(layers=args.layers,
                        max_seq=int(math.ceil((args.prompt + args.generate + 8) / 128) * 128))
    batches = [int(s) for s in args.batch.split(",")]
    shard = None
    if world > 1:
        # torchrun: the TwELL FFN is d_ff-sharded over the ranks, the shard sum runs inside the
        # contraction kernel for decode steps and through the peer all-reduce / NCCL for prefill
        from . import peer_allreduce
        shard = {"rank": rank, "world": world,
                 "peer_allreduce": peer_allreduce.PeerAllReduce(max(batches) * cfg.d_model * 2,
                                                                device=dev),
                 "fused_allreduce": peer_allreduce.FusedShardAllReduce(max(batches), cfg.d_model,
                                                                       device=dev)}
    for b in batches:
        rec = {"batch": b, "n_gpus": world, "prompt": args.prompt, "generate": args.generate,
               "layers": cfg.layers, "d_model": cfg.d_model, "d_ff": cfg.d_ff, "heads": cfg.heads,
               "vocab": cfg.vocab, "gate_density": cfg.density, "dtype": "bf16",
               "data": "synthetic"}
        rec["twell"] = time_decode(cfg, b, args.prompt, args.generate, "twell", shard=shard)
        if rank == 0:  # the comparison point is the unsharded dense-FFN model on one GPU
            rec["dense"] = time_decode(cfg, b, args.prompt, args.generate, "dense")
            rec["speedup_vs_dense_ffn"] = rec["dense"]["ms_per_token"] / rec["twell"]["ms_per_token"]
            if shard is not None:
                rec["allreduce_status"] = [shard["peer_allreduce"].status(),
                                           shard["fused_allreduce"].status()]
            print(json.dumps(rec), flush=True)
        if world > 1:
            torch.cuda.synchronize(dev)
            dist.barrier()
    if world > 1:
        sys.stdout.flush()
        os._exit(0)  # captured graphs hold communicator state: skip the collective teardown


if __name__ == "__main__":
    main()
