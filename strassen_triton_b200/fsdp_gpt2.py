"""GPT-2-small train step under FSDP with every Linear routed through the B200 matmul library.

Offline stand-in for the reference's modded-nanogpt FSDP scripts
(modded_nanogpt/fsdp_train_gpt2.py:650-670: FSDP per Block, bf16 MixedPrecision, use_orig_params;
modded_nanogpt/data_dist_train_gpt2.py:327-389: LinearStrassen for q/k/v/proj and both MLP linears):
same model shape and wrap recipe, random uniform token ids instead of the fineweb shards, AdamW
instead of Muon, no wandb/optuna, plain causal attention. It exists to exercise LinearStrassen
(forward and backward through libb200s.so) under FSDP's flat parameters, all-gather and
reduce-scatter.

    torchrun --nproc-per-node 8 -m strassen_triton_b200.fsdp_gpt2 --steps 10
    python -m strassen_triton_b200.fsdp_gpt2 --layers 2 --steps 3          # one GPU

The reference's training configuration at GPT-2-124M size: 12 layers, d = 768, 12 heads, vocab 50257 (padded to 50304 rows so that every
matrix row is a whole number of 16-byte vectors), sequence 1024, 8 sequences per GPU.
"""
from __future__ import annotations

import argparse
import functools
import math
import os
import time

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
from torch.distributed.fsdp import MixedPrecision
from torch.distributed.fsdp.wrap import transformer_auto_wrap_policy

from .linear import LinearStrassen

VOCAB = 50257
VOCAB_PADDED = 50304


def _linear_factory(depth, device, plain: bool):
    """LinearStrassen (the library's kernels), or nn.Linear for the twin model of the check."""
    if plain:
        return functools.partial(nn.Linear, bias=False, device=device)
    return functools.partial(LinearStrassen, bias=False, depth=depth, device=device)


class Block(nn.Module):
    def __init__(self, d: int, heads: int, depth, device, plain: bool = False):
        super().__init__()
        mk = _linear_factory(depth, device, plain)
        self.heads = heads
        self.ln1 = nn.LayerNorm(d, device=device)
        self.ln2 = nn.LayerNorm(d, device=device)
        self.qkv = mk(d, 3 * d)       # X[8192,768] . W[768,2304]
        self.proj = mk(d, d)
        self.fc = mk(d, 4 * d)        # X[8192,768] . W[768,3072]
        self.out = mk(4 * d, d)       # X[8192,3072] . W[3072,768]

    def forward(self, x):
        b, t, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, t, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, t, d))
        return x + self.out(F.gelu(self.fc(self.ln2(x))))


class GPT(nn.Module):
    def __init__(self, layers=12, d=768, heads=12, seq=1024, depth=None, device="cuda", plain: bool = False):
        super().__init__()
        self.wte = nn.Embedding(VOCAB_PADDED, d, device=device)
        self.wpe = nn.Embedding(seq, d, device=device)
        self.blocks = nn.ModuleList(Block(d, heads, depth, device, plain) for _ in range(layers))
        self.ln_f = nn.LayerNorm(d, device=device)
        self.lm_head = _linear_factory(depth, device, plain)(d, VOCAB_PADDED)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)

    def forward(self, idx, targets):
        t = idx.shape[1]
        x = self.wte(idx) + self.wpe(torch.arange(t, device=idx.device))
        for blk in self.blocks:
            x = blk(x)
        logits = self.lm_head(self.ln_f(x))
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))


def build(layers, seq, depth, device, world, plain: bool = False, state=None):
    model = GPT(layers=layers, seq=seq, depth=depth, device=device, plain=plain)
    if state is not None:
        model.load_state_dict(state)
    if world == 0:
        return model.to(torch.bfloat16)
    mp = MixedPrecision(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16, buffer_dtype=torch.bfloat16)
    policy = functools.partial(transformer_auto_wrap_policy, transformer_layer_cls={Block})
    return FSDP(model, auto_wrap_policy=policy, mixed_precision=mp, use_orig_params=True,
                device_id=torch.cuda.current_device(), sync_module_states=world > 1)


def train_steps(model, steps, batch, seq, rank, lr=3e-4):
    """Runs `steps` optimizer steps on random tokens; returns the list of losses."""
    opt = torch.optim.AdamW(model.parameters(), lr=lr, weight_decay=0.0)
    g = torch.Generator(device="cuda").manual_seed(rank)
    losses = []
    for _ in range(steps):
        ids = torch.randint(0, VOCAB, (batch, seq + 1), generator=g, device="cuda")
        loss = model(ids[:, :-1], ids[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        losses.append(loss.item())
    return losses


def twin_check(world, rank, layers=2, seq=256, batch=4):
    """The FSDP smoke check: a `layers`-layer model whose Linears are LinearStrassen and a twin with
    nn.Linear holding the same weights take one forward/backward on the same tokens under the same
    FSDP wrapping; their losses and every local gradient shard must agree within the tolerance of a
    bf16 product computed by two different kernels. Returns (ok, details)."""
    torch.manual_seed(1234)
    base = GPT(layers=layers, seq=seq, depth=None, device="cuda")
    state = {k: v.clone() for k, v in base.state_dict().items()}
    del base
    ours = build(layers, seq, None, "cuda", world, plain=False, state=state)
    twin = build(layers, seq, None, "cuda", world, plain=True, state=state)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    ids = torch.randint(0, VOCAB, (batch, seq + 1), generator=g, device="cuda")
    losses, grads = [], []
    for model in (ours, twin):
        loss = model(ids[:, :-1], ids[:, 1:])
        loss.backward()
        losses.append(loss.item())
        grads.append({n: p.grad.detach().float().clone() for n, p in model.named_parameters()
                      if p.grad is not None and p.grad.numel() > 0})
    worst, worst_name = 0.0, ""
    for name, g_ours in grads[0].items():
        g_twin = grads[1].get(name)
        if g_twin is None or g_twin.shape != g_ours.shape:
            return False, {"error": f"gradient shard of {name} has no twin"}
        denom = g_twin.norm().item()
        if denom == 0.0:
            continue
        rel = ((g_ours - g_twin).norm().item()) / denom
        if rel > worst:
            worst, worst_name = rel, name
    dloss = abs(losses[0] - losses[1])
    ok = bool(worst < 3e-2 and dloss < 2e-2 and len(grads[0]) > 0 and all(math.isfinite(x) for x in losses))
    return ok, {"layers": layers, "loss_ours": round(losses[0], 4), "loss_twin": round(losses[1], 4),
                "worst_grad_rel_fro": round(worst, 5), "worst_param": worst_name, "grad_shards_compared": len(grads[0]),
                "tolerance": "loss 2e-2, gradients 3e-2 relative Frobenius (bf16 products from two kernels)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=8, help="sequences per GPU")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--depth", type=int, default=-1, help="Strassen depth of the Linears (-1 = tuner table)")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if not dist.is_initialized():
        if "MASTER_ADDR" not in os.environ:
            os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", "29533"
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    from . import _lib

    model = build(args.layers, args.seq, None if args.depth < 0 else args.depth, "cuda", world)
    train_steps(model, 2, args.batch, args.seq, rank)          # warm-up
    torch.cuda.synchronize()
    launches = _lib.load().b200s_launch_count()
    t0 = time.perf_counter()
    losses = train_steps(model, args.steps, args.batch, args.seq, rank)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    if rank == 0:
        tok = world * args.batch * args.seq * args.steps / dt
        print(f"world {world} layers {args.layers}: loss {losses[0]:.3f} -> {losses[-1]:.3f}, "
              f"{dt / args.steps * 1e3:.1f} ms/step, {tok:,.0f} tokens/s, "
              f"{(_lib.load().b200s_launch_count() - launches) // args.steps} library launches per step")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
