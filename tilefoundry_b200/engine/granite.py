"""granite-4.0-h decode session: Mamba-2 state and convolution windows updated in place, paged KV for the
attention layers, expert weights left in their authored ``[experts, ...]`` slabs (rows gathered on the
device by the routing indices), one captured step."""
from __future__ import annotations

import ctypes as C

import torch

from .. import lib
from ..authored.granite_4_0_h_small import GraniteConfig
from . import paged_kv, sharding
from .session import DecodeSession

MAMBA_W = ("gamma_in", "w_in", "conv_w", "conv_b", "a_log", "dt_bias", "d_skip", "gamma_ssm", "w_out")
ATTN_W = ("gamma_in", "w_q", "w_k", "w_v", "w_o")
MOE_W = ("gamma_post", "w_gate", "w_up", "w_down", "w_shared_in", "w_shared_out")


def pack_mixer(kind: str, w: dict) -> dict:
    if kind == "linear_attention":
        return {n: w[n].contiguous() for n in MAMBA_W}
    return {"gamma_in": w["gamma_in"].contiguous(), "w_in": torch.cat([w["w_q"], w["w_k"], w["w_v"]], 0).contiguous(),
            "w_out": w["w_o"].contiguous()}


def pack_model(cfg: GraniteConfig, resource, device=None):
    """Authored names -> kernel layout of the whole model, unsharded (``engine/packed_models.py`` ``PackedModel``)."""
    from .packed_models import PackedModel
    to = (lambda t: t) if device is None else (lambda t: t.to(device))
    root = {"table": to(resource.load("table")).contiguous(), "gamma_final": to(resource.load("gamma_final")).contiguous()}
    layers = []
    for i, kind in enumerate(cfg.layer_types):
        sub = resource.subtree(f"layer{i}")
        mix, moe = sub.subtree("mixer"), sub.subtree("moe")
        names = MAMBA_W if kind == "linear_attention" else ATTN_W
        layer = pack_mixer(kind, {n: to(mix.load(n)) for n in names})
        layer.update({n: to(moe.load(n)).contiguous() for n in MOE_W})
        layer["w_router"] = to(moe.subtree("router").load("w_router")).contiguous()
        layers.append(layer)
    return PackedModel("granite_4_0_h_small", root, layers)


def shard_layer(layer: dict, rank: int, world: int) -> dict:
    """This rank's part of a packed layer: its experts (``e % world == rank``), its slice of the shared expert; the
    mixer, the norms and the router stay whole."""
    out = dict(layer)
    for n in ("w_gate", "w_up", "w_down"):
        out[n] = sharding.local_experts(layer[n], rank, world)
    out["w_shared_in"], out["w_shared_out"] = sharding.shared_slices(layer["w_shared_in"], layer["w_shared_out"], rank, world)
    return out


class GraniteSession(DecodeSession):
    def __init__(self, cfg: GraniteConfig, resource, *, max_ctx: int = 2176, device="cuda:0",
                 keep_logits: bool = False, trace_hidden: bool = False, pdl: bool = True, group=None,
                 collectives: str | None = None, temperature: float = 0.0, seed: int = 0):
        """*group*: a ``torch.distributed`` process group (NCCL) to shard the MoE blocks and the head over;
        ``None`` runs everything on this GPU.  *collectives*: ``"peer"`` = the two exchange steps as single kernels
        over NVLink peer memory (symmetric memory), ``"nccl"`` = NCCL all-reduce / all-gather followed by the
        finishing kernels; ``None`` picks ``"peer"`` when symmetric memory can be set up, else ``"nccl"``."""
        if not torch.cuda.is_available():
            raise RuntimeError("GraniteSession needs a CUDA device; there is no CPU path")
        self.group = group
        if group is not None:
            import torch.distributed as dist
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        lib.load()
        self.cfg, self.device, self.max_ctx = cfg, torch.device(device), int(max_ctx)
        dev = self.device
        to = lambda t: t.to(dev)
        from .packed_models import PackedModel
        # a resource speaks the authored names and is packed here (on this device when one rank holds everything,
        # where the tensors lie when the model is sharded, so that only this rank's shard travels); a PackedModel is
        # already in the kernels' layout
        packed = resource if isinstance(resource, PackedModel) else pack_model(cfg, resource, dev if self.world == 1 else None)
        self.table_w = to(packed.root["table"]).contiguous()
        self.gamma_final = to(packed.root["gamma_final"]).contiguous()
        bf, f32 = torch.bfloat16, torch.float32
        z = lambda *s, dtype=bf: torch.zeros(*s, device=dev, dtype=dtype)
        HQ, HKV, D, H = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.hidden_size
        E, K, I, IS, V = (cfg.num_local_experts, cfg.num_experts_per_tok, cfg.intermediate_size,
                          cfg.shared_intermediate_size, cfg.vocab_size)
        self.table = paged_kv.block_table(1, self.max_ctx, device=dev)
        self.layers = []
        for i, kind in enumerate(cfg.layer_types):
            layer = packed.layers[i] if self.world == 1 else shard_layer(packed.layers[i], self.rank, self.world)
            layer = {n: to(t).contiguous() for n, t in layer.items()}
            layer["kind"] = kind
            if kind == "linear_attention":
                layer["conv_state"] = z(cfg.conv_dim, cfg.mamba_d_conv - 1)
                layer["ssm_state"] = z(cfg.mamba_n_heads, cfg.mamba_d_head, cfg.mamba_d_state, dtype=f32)
            else:
                layer["k_pool"] = paged_kv.new_pool(1, self.max_ctx, HKV, D, device=dev)
                layer["v_pool"] = paged_kv.new_pool(1, self.max_ctx, HKV, D, device=dev)
            self.layers.append(layer)

        nsplit = lib.attn_splits(self.max_ctx)
        L = len(self.layers)
        self.tokens, self.pos = z(self.max_ctx + 1, dtype=torch.int64), z(1, dtype=torch.int32)
        self.hidden = z(H)
        self.proj = z(max(cfg.proj, (HQ + 2 * HKV) * D))
        self.mixed = z(cfg.conv_dim)
        self.y = z(max(cfg.expand, HQ * D))
        self.router_logits, self.router_idx, self.router_w = z(E), z(K, dtype=torch.int64), z(K)
        self.inner, self.shared = z(K * I), z(IS)
        self.logits = z(V) if keep_logits else None
        self.part_o, self.part_ml = z(HQ * nsplit * D, dtype=f32), z(HQ * nsplit * 2, dtype=f32)
        self.counters = z(HKV + 1, dtype=torch.int32)
        n_head = lib.lm_head_scratch_entries(V)
        self.head_val, self.head_idx = z(n_head, dtype=f32), z(n_head, dtype=torch.int32)
        self.trace = z(L + 1, H) if trace_hidden else None
        self.idx_trace = z(L, K, dtype=torch.int64) if trace_hidden else None
        self.picked = z(1, dtype=torch.int64)
        self.partial, self.pair, self.gathered = z(2, H, dtype=f32), z(2, dtype=f32), z(self.world, 2, dtype=f32)
        if self.world > 1:
            sharding.vocab_slice(V, self.rank, self.world)          # validates divisibility

        self._layer_structs = (lib.GraniteLayer * L)()
        for s, layer in zip(self._layer_structs, self.layers):
            s.kind = 0 if layer["kind"] == "linear_attention" else 1
            for name, _ in lib.GraniteLayer._fields_[2:]:
                setattr(s, name, lib.ptr(layer.get(name)))
        as_bf16 = lambda v: float(torch.tensor(v, dtype=bf))
        self.args = lib.GraniteStepArgs(
            temperature=float(temperature), seed=int(seed) & (2 ** 64 - 1),
            layers=self._layer_structs, n_layers=L, hidden=H, nh=cfg.mamba_n_heads, pd=cfg.mamba_d_head,
            ns=cfg.mamba_d_state, ng=cfg.mamba_n_groups, conv_width=cfg.mamba_d_conv, hq=HQ, hkv=HKV, d=D,
            experts=E, top_k=K, inter=I, shared_inter=IS, vocab=V, eps=cfg.rms_norm_eps,
            attn_scale=cfg.attention_multiplier, embed_scale=as_bf16(cfg.embedding_multiplier),
            res_scale=as_bf16(cfg.residual_multiplier), logits_scale=1.0 / cfg.logits_scaling,
            table=lib.ptr(self.table_w), gamma_final=lib.ptr(self.gamma_final), page_size=paged_kv.PAGE_SIZE,
            table_len=self.table.shape[1], max_ctx=self.max_ctx, block_table=lib.ptr(self.table),
            tokens=lib.ptr(self.tokens), pos=lib.ptr(self.pos), n_prompt=0, max_tokens=self.max_ctx + 1,
            hidden_buf=lib.ptr(self.hidden), proj_buf=lib.ptr(self.proj), mixed_buf=lib.ptr(self.mixed),
            y_buf=lib.ptr(self.y), router_logits=lib.ptr(self.router_logits), router_idx=lib.ptr(self.router_idx),
            router_w=lib.ptr(self.router_w), inner_buf=lib.ptr(self.inner), shared_buf=lib.ptr(self.shared),
            logits=lib.ptr(self.logits), part_o=lib.ptr(self.part_o), part_ml=lib.ptr(self.part_ml),
            counters=lib.ptr(self.counters), head_val=lib.ptr(self.head_val), head_idx=lib.ptr(self.head_idx),
            hidden_trace=lib.ptr(self.trace), idx_trace=lib.ptr(self.idx_trace), picked=lib.ptr(self.picked),
            pdl=int(pdl), ep_rank=self.rank, ep_world=self.world, partial=lib.ptr(self.partial),
            pair=lib.ptr(self.pair), gathered=lib.ptr(self.gathered))
        self.collectives = "none"
        if self.world > 1:
            self.collectives = self._setup_peer_exchange(H, collectives)
        n_m = sum(1 for l in self.layers if l["kind"] == "linear_attention")
        self.launches_per_step = 2 + 9 * n_m + 8 * (L - n_m) + (2 * L + 1 if trace_hidden else 0) + (
            L + 1 if self.world > 1 else 0)              # sharded: one finalize per layer and the final pick

    def _setup_peer_exchange(self, H: int, want: str | None) -> str:
        """Argument blocks of the two exchange kernels over the ranks' symmetric buffers.  Returns the mode in use."""
        from .peer import PeerBuffers
        self._peer = PeerBuffers(self.group, self.rank, self.world, H, self.device, want)
        if self._peer.mode != "peer":
            return self._peer.mode
        pb, W, a = self._peer, self.world, self.args
        self.peer_epoch, self.pick_epoch, self.peer_status = pb.reduce_epoch, pb.pick_epoch, pb.status
        self._reduce_args = lib.MoeAllreduceArgs(
            partial=lib.ptr(self.partial), epoch=lib.ptr(pb.reduce_epoch), status=lib.ptr(pb.status),
            residual=lib.ptr(self.hidden), out=lib.ptr(self.hidden), hidden=H, rank=self.rank, world=W, has_shared=1,
            res_scale=a.res_scale, pdl=a.pdl)
        self._pick_args = lib.PickAllgatherArgs(
            pair=lib.ptr(self.pair), epoch=lib.ptr(pb.pick_epoch), status=lib.ptr(pb.status),
            tokens=lib.ptr(self.tokens), pos=lib.ptr(self.pos), picked=lib.ptr(self.picked), n_prompt=0,
            max_tokens=self.max_ctx + 1, rank=self.rank, world=W, pdl=a.pdl)
        for r in range(W):
            self._reduce_args.inbox[r], self._reduce_args.flags[r] = pb.reduce_inbox[r], pb.reduce_flags[r]
            self._pick_args.inbox[r], self._pick_args.flags[r] = pb.pick_inbox[r], pb.pick_flags[r]
        return "peer"

    def reset(self, prompt_ids) -> None:
        super().reset(prompt_ids)
        if self.collectives == "peer":
            import torch.distributed as dist
            self._pick_args.n_prompt = self.args.n_prompt
            torch.cuda.synchronize()
            dist.barrier(group=self.group)           # the ranks' kernels wait on one another: start them together
        for layer in self.layers:                    # recurrent state starts at zero for a new sequence
            if layer["kind"] == "linear_attention":
                layer["conv_state"].zero_()
                layer["ssm_state"].zero_()

    def state_tensors(self) -> list:
        return [l[n] for l in self.layers if l["kind"] == "linear_attention" for n in ("conv_state", "ssm_state")]

    def weight_bytes(self) -> int:
        """Bytes of weights one token reads: every mixer, router and shared expert, top-k experts, the head."""
        cfg, total = self.cfg, self.table_w.numel() * 2
        for l in self.layers:
            total += (l["w_in"].numel() + l["w_out"].numel() + l["w_router"].numel() + l["w_shared_in"].numel()
                      + l["w_shared_out"].numel()) * 2
            total += cfg.num_experts_per_tok * 3 * cfg.intermediate_size * cfg.hidden_size * 2 // self.world
        if self.world > 1:                           # the head is sliced too; the table is read for one row
            total -= self.table_w.numel() * 2 * (self.world - 1) // self.world
        return total

    def state_bytes(self) -> int:
        n_m = sum(1 for l in self.layers if l["kind"] == "linear_attention")
        c = self.cfg
        return n_m * 2 * c.mamba_n_heads * c.mamba_d_head * c.mamba_d_state * 4

    def kv_bytes_per_position(self) -> int:
        c = self.cfg
        return 2 * c.num_key_value_heads * c.head_dim * 2 * len(c.attention_layers)

    def step(self) -> None:
        if self.world == 1:
            lib.check(lib.load().tfb_granite_decode_step(C.byref(self.args), lib.stream()), "tfb_granite_decode_step")
            return
        import torch.distributed as dist
        part = lambda p, l=0: lib.check(lib.load().tfb_granite_step_part(C.byref(self.args), p, l, lib.stream()),
                                        "tfb_granite_step_part")
        peer = self.collectives == "peer"
        part(0)
        for l in range(len(self.layers)):
            part(1, l)
            if peer:                                                 # exchange + finish in one kernel over NVLink
                lib.check(lib.load().tfb_moe_allreduce_finalize(C.byref(self._reduce_args), lib.stream()),
                          "tfb_moe_allreduce_finalize")
            else:
                dist.all_reduce(self.partial, group=self.group)      # one reduction per MoE block
                part(2, l)
        part(3)
        if peer:
            lib.check(lib.load().tfb_pick_allgather(C.byref(self._pick_args), lib.stream()), "tfb_pick_allgather")
        else:
            dist.all_gather_into_tensor(self.gathered, self.pair, group=self.group)
            part(4)
