"""Run under torchrun (one rank per GPU): the sharded granite session must produce the single-GPU session's
tokens and logits.  Rank 0 prints `MULTI_GPU_OK` on success.  Used by tests/test_multi_gpu.py."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from tilefoundry_b200.authored import granite_4_0_h_small as gr          # noqa: E402
from tilefoundry_b200.authored.weights import random_weights            # noqa: E402
from tilefoundry_b200.engine.granite import GraniteSession              # noqa: E402
from tilefoundry_b200.runtime import DictResource                       # noqa: E402


def say(*a):
    print(f"[rank {os.environ.get('RANK', '?')}]", *a, file=sys.stderr, flush=True)


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")                     # plain peer stores only: no NVLink multicast binding
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    probe = torch.ones(4, device=dev)
    dist.all_reduce(probe)
    torch.cuda.synchronize()
    say("nccl up", probe.tolist())
    cfg = gr.GRANITE_TINY
    weights = random_weights(gr.build(cfg), seed=11, std=0.05, overrides=gr.weight_overrides)
    on_dev = {k: v.to(dev) for k, v in weights.items()}
    prompt = torch.randint(0, cfg.vocab_size, (16,), generator=torch.Generator().manual_seed(3))
    n_new = 70
    single = GraniteSession(cfg, DictResource(on_dev), max_ctx=100, device=dev, keep_logits=True)
    want = single.generate(prompt, n_new, use_graph=False).tokens
    want_logits = single.logits.clone()
    say("single-GPU reference done")
    modes = []
    for mode in ("nccl", "peer"):                     # NCCL collectives, then the single-kernel exchange over peer memory
        try:
            sharded = GraniteSession(cfg, DictResource(on_dev), max_ctx=100, device=dev, keep_logits=True,
                                     group=dist.group.WORLD, collectives=mode)
        except RuntimeError as exc:
            say(f"mode {mode} unavailable: {exc}")
            continue
        modes.append(mode)
        for use_graph in (False, True):
            say("sharded generate, graph =", use_graph)
            got = sharded.generate(prompt, n_new, use_graph=use_graph).tokens
            say("done")
            full = torch.zeros_like(sharded.logits)
            per = cfg.vocab_size // world
            full[rank * per:(rank + 1) * per] = sharded.logits[rank * per:(rank + 1) * per]
            dist.all_reduce(full)
            same = sum(a == b for a, b in zip(got, want))
            err = float((full.float() - want_logits.float()).abs().max())
            scale = float(want_logits.float().abs().max())
            # tokens: identical unless an f32 summation-order difference flips a bf16 rounding on a near-tie
            assert got[:8] == want[:8], (got[:8], want[:8])
            assert same >= n_new - 2 or got == want, f"{same}/{n_new} tokens equal"
            if got == want:
                assert err <= 2e-2 + 2e-2 * scale, f"logits differ by {err} (scale {scale})"
            picks = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(world)]
            dist.all_gather(picks, sharded.picked)
            assert all(int(p) == int(picks[0]) for p in picks), "ranks disagree on the picked token"
        if mode == "peer":
            assert int(sharded.peer_status) == 0, f"a bounded peer wait gave up: {int(sharded.peer_status):#x}"
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print(f"MULTI_GPU_OK world={world} modes={modes} tokens_equal={same}/{n_new} logit_err={err:.4g}", flush=True)
    # graphs that recorded NCCL kernels keep the communicator alive: they are dropped before the teardown
    from tilefoundry_b200.engine.peer import leave_together
    leave_together([single, sharded])


if __name__ == "__main__":
    main()
