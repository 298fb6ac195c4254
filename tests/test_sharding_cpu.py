"""The multi-GPU split of a MoE block and of the head, checked on the CPU with two gloo ranks.

Each rank takes its shard exactly as `GraniteSession` does (`engine/sharding.py`), computes its partial
sums in torch with the kernels' rounding points, the ranks all-reduce / all-gather, and the result must
match the unsharded CPU oracle.  The routing indices are computed on every rank and must be identical.
"""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tilefoundry_b200.engine import sharding

BF = torch.bfloat16


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import evaluator, granite_4_0_h_small as og
        from tilefoundry_b200.authored import granite_4_0_h_small as gr
        from tilefoundry_b200.authored.weights import random_weights
        from tilefoundry_b200.runtime import DictResource

        cfg = gr.GRANITE_TINY
        mod = gr.build(cfg)
        weights = random_weights(mod, seed=5, std=0.05, overrides=gr.weight_overrides)
        ref = evaluator.load(mod, DictResource(weights), og.make(cfg))
        moe = ref.layer0.moe
        hidden = torch.randn(1, 1, cfg.hidden_size, generator=torch.Generator().manual_seed(1)).to(BF)
        tokens = moe.post_norm(hidden)
        w, idx = moe.router.routing(tokens)                       # replicated router: same on every rank
        gathered_idx = [torch.zeros_like(idx) for _ in range(world)]
        dist.all_gather(gathered_idx, idx)
        assert all(torch.equal(g, idx) for g in gathered_idx)

        c = moe.constants
        K, I, H = cfg.num_experts_per_tok, cfg.intermediate_size, cfg.hidden_size
        gate_l, up_l, down_l = (sharding.local_experts(c[n], rank, world) for n in ("w_gate", "w_up", "w_down"))
        sh_in, sh_out = sharding.shared_slices(c["w_shared_in"], c["w_shared_out"], rank, world)
        x = tokens.reshape(H)
        routed = torch.zeros(H, dtype=torch.float32)
        for s in range(K):
            e = int(idx[0, s])
            if sharding.expert_owner(e, world) != rank:
                continue
            le = e // world
            inner = torch.nn.functional.silu(gate_l[le] @ x) * (up_l[le] @ x)          # bf16 ops round like the kernel
            routed += ((down_l[le] @ inner) * w[0, s]).float()
        per = sh_in.shape[0] // 2
        act = torch.nn.functional.silu(sh_in[:per] @ x) * (sh_in[per:] @ x)
        shared = sh_out.float() @ act.float()                                           # un-rounded partial dot
        partial = torch.stack([routed, shared])
        dist.all_reduce(partial)
        res = torch.randn(H, generator=torch.Generator().manual_seed(2)).to(BF)
        scale = torch.tensor(cfg.residual_multiplier, dtype=BF)
        e_out = partial[0].to(BF) + partial[1].to(BF)
        got = res + e_out * scale
        want = ref.layer0.residual_add(res.reshape(1, 1, H), moe.experts(tokens, w, idx)).reshape(H)
        err = (got.float() - want.float()).abs().max().item()
        bound = 2e-2 + 2e-2 * want.float().abs().max().item()

        # vocabulary-parallel pick
        logits = ref.lm_head(ref.final_rms_norm(hidden))[0]
        lo, hi = sharding.vocab_slice(cfg.vocab_size, rank, world)
        local = logits[lo:hi].float()
        pair = torch.tensor([float(local.max()), float(lo + int(torch.argmax(local)))])
        pairs = [torch.zeros(2) for _ in range(world)]
        dist.all_gather(pairs, pair)
        pick = sharding.pick_from_pairs(torch.stack(pairs))
        out[rank] = (err, bound, pick, int(torch.argmax(logits)))
    finally:
        dist.destroy_process_group()


def test_two_rank_moe_block_and_vocab_parallel_pick():
    world = 2
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(world, 29531 + os.getpid() % 200, out), nprocs=world, join=True)
    assert len(out) == world
    for rank in range(world):
        err, bound, pick, want_pick = out[rank]
        assert err <= bound, f"rank {rank}: sharded MoE block differs by {err:.4g} > {bound:.4g}"
        assert pick == want_pick


def test_sharding_helpers_reject_uneven_splits():
    w = torch.zeros(9, 4, 4)
    with pytest.raises(ValueError, match="do not divide"):
        sharding.local_experts(w, 0, 2)
    assert sharding.local_experts(torch.arange(8).reshape(8, 1), 1, 4).flatten().tolist() == [1, 5]
    with pytest.raises(ValueError, match="does not divide"):
        sharding.vocab_slice(1001, 0, 2)
    with pytest.raises(ValueError, match="multiples of 8"):
        sharding.shared_slices(torch.zeros(24, 8), torch.zeros(8, 12), 0, 2)
    assert sharding.pick_from_pairs(torch.tensor([[1.0, 700.0], [1.0, 20.0], [0.5, 3.0]])) == 20


def _worker_qwen35(rank, world, port, out):
    """The f32-activation MoE block (Qwen3.5) split the way `Qwen35Session` splits it: every rank computes, with the
    kernels' rounding points, the routed sum of the experts it owns and its slice's un-rounded shared dot; the sums
    are added across ranks before the shared expert's single rounding and its sigmoid gate are applied."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import evaluator, qwen3_5_35b_a3b as oq
        from tilefoundry_b200.authored import qwen3_5_35b_a3b as qa
        from tilefoundry_b200.authored.weights import random_weights
        from tilefoundry_b200.runtime import DictResource

        cfg = qa.QWEN3_5_TINY
        mod = qa.build(cfg)
        weights = random_weights(mod, seed=5, std=0.05, overrides=qa.weight_overrides)
        ref = evaluator.load(mod, DictResource(weights), oq.make(cfg))
        moe = ref.layer0.moe
        attended = torch.randn(1, 1, cfg.hidden, generator=torch.Generator().manual_seed(1))
        tokens = moe.post_norm(attended)
        w, idx = moe.router.routing(tokens)                       # replicated router: same on every rank
        gathered_idx = [torch.zeros_like(idx) for _ in range(world)]
        dist.all_gather(gathered_idx, idx)
        assert all(torch.equal(g, idx) for g in gathered_idx)

        c = moe.constants
        K, IS, H = cfg.top_k, cfg.shared_intermediate, cfg.hidden
        mm = lambda a, b: torch.matmul(a.to(BF), b.to(BF)).float()  # a product: bf16 in, bf16 out, carried as f32
        gate_l, up_l, down_l = (sharding.local_experts(c[n], rank, world) for n in ("w_gate", "w_up", "w_down"))
        x = tokens.reshape(H)
        routed = torch.zeros(H)
        for s in range(K):
            e = int(idx[0, s])
            if sharding.expert_owner(e, world) != rank:
                continue
            le = e // world
            inner = torch.nn.functional.silu(mm(gate_l[le], x)) * mm(up_l[le], x)
            routed += mm(down_l[le], inner) * w[0, s]
        per = IS // world
        lo, hi = rank * per, (rank + 1) * per
        act = (torch.nn.functional.silu(mm(x, c["w_shared_gate"][:, lo:hi])) * mm(x, c["w_shared_up"][:, lo:hi])).to(BF)
        shared = act.float() @ c["w_shared_down"][lo:hi, :].float()                     # un-rounded partial dot
        partial = torch.stack([routed, shared])
        dist.all_reduce(partial)
        gate = torch.sigmoid(mm(x, c["w_shared_scale"]))
        got = attended.reshape(H) + partial[0] + partial[1].to(BF).float() * gate
        want = ref.layer0.residual_add(attended, moe.experts(tokens, w, idx)).reshape(H)
        err = (got - want).abs().max().item()
        out[rank] = (err, 2e-2 + 2e-2 * want.abs().max().item())
    finally:
        dist.destroy_process_group()


def test_two_rank_qwen3_5_moe_block():
    world = 2
    out = mp.Manager().dict()
    mp.spawn(_worker_qwen35, args=(world, 29331 + os.getpid() % 200, out), nprocs=world, join=True)
    assert len(out) == world
    for rank in range(world):
        err, bound = out[rank]
        assert err <= bound, f"rank {rank}: sharded Qwen3.5 MoE block differs by {err:.4g} > {bound:.4g}"
