"""Qwen3.5-35B-A3B decode session: f32 hidden state, Gated DeltaNet state and convolution windows updated on
the device, a paged f32 KV cache for the gated-attention layers, expert weights left in their authored
``[experts, ...]`` slabs (rows gathered on the device by the routing indices), one captured step."""
from __future__ import annotations

import ctypes as C

import torch

from .. import lib
from ..authored.qwen3_5_35b_a3b import Qwen35Config, rope_tables
from . import paged_kv, sharding
from .session import DecodeSession


def _rows(w: torch.Tensor) -> torch.Tensor:
    """Authored ``(1, in, out)`` / ``(in, out)`` matrix as ``[out, in]`` rows."""
    return w.reshape(w.shape[-2], w.shape[-1]).t().contiguous()


def pack_mixer(kind: str, w: dict) -> dict:
    """The mixer's projections as row-major ``[out, in]`` slabs, the ones that share an input concatenated."""
    if kind == "linear_attention":
        return {"gamma_in": w["gamma_in"].contiguous(),
                "w_in": torch.cat([_rows(w[n]) for n in ("w_in_qkv", "w_in_z", "w_in_b", "w_in_a")], 0).contiguous(),
                "w_out": _rows(w["w_out"]), "conv_w": w["conv_w"].contiguous(), "a_log": w["a_log"].contiguous(),
                "dt_bias": w["dt_bias"].contiguous(), "gamma_gdn": w["gamma_gdn"].contiguous()}
    return {"gamma_in": w["gamma_in"].contiguous(),
            "w_in": torch.cat([_rows(w[n]) for n in ("w_qg", "w_k", "w_v")], 0).contiguous(),
            "w_out": _rows(w["w_o"]), "gamma_q": w["gamma_q"].contiguous(), "gamma_k": w["gamma_k"].contiguous()}


def pack_moe(w: dict, w_router: torch.Tensor) -> dict:
    return {"gamma_post": w["gamma_post"].contiguous(),
            "w_router": torch.cat([_rows(w_router), _rows(w["w_shared_scale"])], 0).contiguous(),
            "w_gate": w["w_gate"].contiguous(), "w_up": w["w_up"].contiguous(), "w_down": w["w_down"].contiguous(),
            "w_shared_gate": _rows(w["w_shared_gate"]), "w_shared_up": _rows(w["w_shared_up"]),
            "w_shared_down": _rows(w["w_shared_down"])}


GDN_W = ("gamma_in", "w_in_qkv", "w_in_z", "w_in_b", "w_in_a", "conv_w", "a_log", "dt_bias", "gamma_gdn", "w_out")
ATTN_W = ("gamma_in", "w_qg", "w_k", "w_v", "gamma_q", "gamma_k", "w_o")
MOE_W = ("gamma_post", "w_gate", "w_up", "w_down", "w_shared_gate", "w_shared_up", "w_shared_down", "w_shared_scale")


def pack_model(cfg: Qwen35Config, resource, device=None):
    """Authored names -> kernel layout of the whole model, unsharded (``engine/packed_models.py`` ``PackedModel``)."""
    from .packed_models import PackedModel
    to = (lambda t: t) if device is None else (lambda t: t.to(device))
    root = {"table": to(resource.load("table")).contiguous(), "gamma_final": to(resource.load("gamma_final")).contiguous(),
            "w_head": _rows(to(resource.load("w_head")))}                  # authored (hidden, vocab) -> [vocab, hidden]
    layers = []
    for i, kind in enumerate(cfg.layer_types):
        sub = resource.subtree(f"layer{i}")
        mix, moe = sub.subtree("mixer"), sub.subtree("moe")
        names = GDN_W if kind == "linear_attention" else ATTN_W
        layer = pack_mixer(kind, {n: to(mix.load(n)) for n in names})
        layer.update(pack_moe({n: to(moe.load(n)) for n in MOE_W}, to(moe.subtree("router").load("w_router"))))
        layers.append(layer)
    return PackedModel("qwen3_5_35b_a3b", root, layers)


def shard_layer(cfg: Qwen35Config, layer: dict, rank: int, world: int) -> dict:
    """This rank's part of a packed layer: its experts (``e % world == rank``) and its rows of the shared expert's
    gate / up projections with the matching columns of its down projection."""
    out = dict(layer)
    for n in ("w_gate", "w_up", "w_down"):
        out[n] = sharding.local_experts(layer[n], rank, world)
    per = cfg.shared_intermediate // world
    lo, hi = rank * per, (rank + 1) * per
    out["w_shared_gate"], out["w_shared_up"] = layer["w_shared_gate"][lo:hi].contiguous(), layer["w_shared_up"][lo:hi].contiguous()
    out["w_shared_down"] = layer["w_shared_down"][:, lo:hi].contiguous()
    return out


class Qwen35Session(DecodeSession):
    def __init__(self, cfg: Qwen35Config, resource, *, max_ctx: int | None = None, device="cuda:0",
                 keep_logits: bool = False, trace_hidden: bool = False, pdl: bool = True, group=None,
                 collectives: str | None = None, expert_prefetch: bool = False,
                 temperature: float = 0.0, seed: int = 0):
        """*group*: a ``torch.distributed`` process group to shard the MoE blocks (expert e on rank ``e % n``, the
        shared expert sliced) and the head (vocabulary slices) over; ``None`` runs everything on this GPU.  The
        exchange steps run as single kernels over NVLink peer memory (*collectives* ``"peer"``, required).
        *expert_prefetch*: the selection kernel asks L2 for the selected experts' weights (measured 2.5 % slower per
        step on B200, so off by default)."""
        if not torch.cuda.is_available():
            raise RuntimeError("Qwen35Session needs a CUDA device; there is no CPU path")
        self.group = group
        if group is not None:
            import torch.distributed as dist
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        lib.load()
        self.cfg, self.device = cfg, torch.device(device)
        self.max_ctx = int(max_ctx or cfg.max_ctx)
        if self.max_ctx > cfg.max_ctx:
            raise ValueError(f"max_ctx {self.max_ctx} exceeds the rotary tables ({cfg.max_ctx})")
        dev = self.device
        to = lambda t: t.to(dev)
        bf, f32 = torch.bfloat16, torch.float32
        z = lambda *s, dtype=f32: torch.zeros(*s, device=dev, dtype=dtype)
        H, V = cfg.hidden, cfg.vocab
        HQ, HKV, D = cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim
        E, K, I, IS = cfg.n_experts, cfg.top_k, cfg.moe_intermediate, cfg.shared_intermediate
        from .packed_models import PackedModel
        # a resource speaks the authored names and is packed here (on this device when one rank holds everything,
        # where the tensors lie when the model is sharded, so that only this rank's shard travels); a PackedModel is
        # already in the kernels' layout
        packed = resource if isinstance(resource, PackedModel) else pack_model(cfg, resource, dev if self.world == 1 else None)
        self.table_w = to(packed.root["table"]).contiguous()
        self.gamma_final = to(packed.root["gamma_final"]).contiguous()
        head = packed.root["w_head"]                                     # [vocab, hidden]
        if self.world > 1:
            lo, hi = sharding.vocab_slice(V, self.rank, self.world)
            head = head[lo:hi]
        self.w_head = to(head).contiguous()
        cos, sin = rope_tables(cfg, "cpu")
        self.cos, self.sin = to(cos).contiguous(), to(sin).contiguous()
        self.table = paged_kv.block_table(1, self.max_ctx, device=dev)
        self.conv_stride = cfg.conv_dim * (cfg.gdn_conv_kernel - 1)
        self.layers = []
        for i, kind in enumerate(cfg.layer_types):
            layer = packed.layers[i] if self.world == 1 else shard_layer(cfg, packed.layers[i], self.rank, self.world)
            layer = {n: to(t).contiguous() for n, t in layer.items()}
            layer["kind"] = kind
            if kind == "linear_attention":
                layer["conv_state"] = z(2, cfg.conv_dim, cfg.gdn_conv_kernel - 1)
                layer["state"] = z(cfg.gdn_n_v_heads, cfg.gdn_head_k_dim, cfg.gdn_head_v_dim)
            else:
                layer["k_pool"] = paged_kv.new_pool(1, self.max_ctx, HKV, D, device=dev, dtype=f32)
                layer["v_pool"] = paged_kv.new_pool(1, self.max_ctx, HKV, D, device=dev, dtype=f32)
            self.layers.append(layer)

        nsplit = lib.load().tfb_attn_gated_splits(self.max_ctx)
        L = len(self.layers)
        self.tokens, self.pos = z(self.max_ctx + 1, dtype=torch.int64), z(1, dtype=torch.int32)
        self.hidden, self.attended = z(H), z(H)
        self.proj = z(max(cfg.conv_dim + cfg.val_dim + 2 * cfg.gdn_n_v_heads, 2 * HQ * D + 2 * HKV * D))
        self.mixed = z(max(cfg.val_dim, HQ * D))
        self.router_logits, self.router_idx, self.router_w = z(E + 1), z(K, dtype=torch.int64), z(K)
        self.inner = z(K * I + IS)
        self.logits = z(V, dtype=bf) if keep_logits else None
        self.part_o, self.part_ml = z(HQ * nsplit * D), z(HQ * nsplit * 2)
        self.counters = z(lib.load().tfb_attn_gated_groups(HQ, HKV, D) + 1, dtype=torch.int32)   # attention tickets, head ticket
        n_head = lib.lm_head_scratch_entries(V)
        self.head_val, self.head_idx = z(n_head), z(n_head, dtype=torch.int32)
        self.trace = z(L + 1, H) if trace_hidden else None
        self.idx_trace = z(L, K, dtype=torch.int64) if trace_hidden else None
        self.picked = z(1, dtype=torch.int64)
        self.partial, self.pair = z(2, H), z(2)
        if self.world > 1 and (IS % self.world or (IS // self.world) % 8):
            raise ValueError(f"shared intermediate size {IS} does not slice over {self.world} ranks in multiples of 8")

        self._layer_structs = (lib.Qwen35Layer * L)()
        for s, layer in zip(self._layer_structs, self.layers):
            s.kind = 0 if layer["kind"] == "linear_attention" else 1
            for name, _ in lib.Qwen35Layer._fields_[2:]:
                setattr(s, name, lib.ptr(layer.get(name)))
        self.args = lib.Qwen35StepArgs(
            temperature=float(temperature), seed=int(seed) & (2 ** 64 - 1),
            layers=self._layer_structs, n_layers=L, pdl=int(pdl), table=lib.ptr(self.table_w),
            gamma_final=lib.ptr(self.gamma_final), w_head=lib.ptr(self.w_head), cos_table=lib.ptr(self.cos),
            sin_table=lib.ptr(self.sin), tokens=lib.ptr(self.tokens), pos=lib.ptr(self.pos), n_prompt=0,
            max_tokens=self.max_ctx + 1, block_table=lib.ptr(self.table), page_size=paged_kv.PAGE_SIZE,
            table_len=self.table.shape[1], max_ctx=self.max_ctx, hidden=H, vocab=V, hk=cfg.gdn_n_k_heads,
            hv=cfg.gdn_n_v_heads, dk=cfg.gdn_head_k_dim, dv=cfg.gdn_head_v_dim, conv_width=cfg.gdn_conv_kernel, hq=HQ,
            hkv=HKV, d=D, rotary_dim=cfg.rotary_dim, experts=E, top_k=K, inter=I, shared_inter=IS,
            conv_state_stride=self.conv_stride, eps=cfg.rms_eps, attn_scale=D ** -0.5, q_scale=cfg.gdn_head_k_dim ** -0.5,
            hidden_buf=lib.ptr(self.hidden), attended_buf=lib.ptr(self.attended), proj_buf=lib.ptr(self.proj),
            mixed_buf=lib.ptr(self.mixed), router_logits=lib.ptr(self.router_logits), router_idx=lib.ptr(self.router_idx),
            router_w=lib.ptr(self.router_w), inner_buf=lib.ptr(self.inner), part_o=lib.ptr(self.part_o),
            part_ml=lib.ptr(self.part_ml), counters=lib.ptr(self.counters), head_val=lib.ptr(self.head_val),
            head_idx=lib.ptr(self.head_idx), logits=lib.ptr(self.logits), picked=lib.ptr(self.picked),
            hidden_trace=lib.ptr(self.trace), idx_trace=lib.ptr(self.idx_trace), ep_rank=self.rank, ep_world=self.world,
            partial=lib.ptr(self.partial), pair=lib.ptr(self.pair), expert_prefetch=int(expert_prefetch))
        self.collectives = "none"
        if self.world > 1:
            from .peer import PeerBuffers
            self._peer = pb = PeerBuffers(self.group, self.rank, self.world, H, dev, "peer" if collectives is None else collectives)
            if pb.mode != "peer":
                raise RuntimeError("the sharded Qwen3.5 step needs peer-memory collectives (symmetric memory)")
            self.collectives, self.peer_status = "peer", pb.status
            self._reduce_args = lib.MoeAllreduceArgs(
                partial=lib.ptr(self.partial), epoch=lib.ptr(pb.reduce_epoch), status=lib.ptr(pb.status), hidden=H,
                rank=self.rank, world=self.world, has_shared=1, res_scale=1.0, pdl=int(pdl),
                residual_f32=lib.ptr(self.attended), out_f32=lib.ptr(self.hidden),
                gate_logit=self.router_logits.data_ptr() + 4 * E)
            self._pick_args = lib.PickAllgatherArgs(
                pair=lib.ptr(self.pair), epoch=lib.ptr(pb.pick_epoch), status=lib.ptr(pb.status), tokens=lib.ptr(self.tokens),
                pos=lib.ptr(self.pos), picked=lib.ptr(self.picked), n_prompt=0, max_tokens=self.max_ctx + 1,
                rank=self.rank, world=self.world, pdl=int(pdl))
            for r in range(self.world):
                self._reduce_args.inbox[r], self._reduce_args.flags[r] = pb.reduce_inbox[r], pb.reduce_flags[r]
                self._pick_args.inbox[r], self._pick_args.flags[r] = pb.pick_inbox[r], pb.pick_flags[r]
        self.launches_per_step = 2 + 7 * L + (2 * L + 1 if trace_hidden else 0) + (L + 1 if self.world > 1 else 0)

    def _recurrent(self):
        return [l for l in self.layers if l["kind"] == "linear_attention"]

    def reset(self, prompt_ids) -> None:
        super().reset(prompt_ids)
        if self.world > 1:
            import torch.distributed as dist
            self._pick_args.n_prompt = self.args.n_prompt
            torch.cuda.synchronize()
            dist.barrier(group=self.group)           # the ranks' kernels wait on one another: start them together
        for layer in self._recurrent():               # recurrent state starts at zero for a new sequence
            layer["conv_state"].zero_()
            layer["state"].zero_()

    def state_tensors(self) -> list:
        return [l[n] for l in self._recurrent() for n in ("conv_state", "state")]

    def conv_window(self, layer: dict) -> torch.Tensor:
        """The convolution window the NEXT step will read, ``[channels, width-1]``."""
        return layer["conv_state"][int(self.pos.item()) & 1]

    def weight_bytes(self) -> int:
        """Bytes of weights one token reads: every mixer, router and shared expert, top-k experts, the head."""
        cfg, total = self.cfg, self.w_head.numel() * 2
        for l in self.layers:
            total += (l["w_in"].numel() + l["w_out"].numel() + l["w_router"].numel() + l["w_shared_gate"].numel()
                      + l["w_shared_up"].numel() + l["w_shared_down"].numel()) * 2
            total += cfg.top_k * 3 * cfg.moe_intermediate * cfg.hidden * 2 // self.world
        return total

    def state_bytes(self) -> int:
        """Recurrent state read and written per token."""
        c = self.cfg
        return len(self._recurrent()) * 2 * c.gdn_n_v_heads * c.gdn_head_k_dim * c.gdn_head_v_dim * 4

    def kv_bytes_per_position(self) -> int:
        c = self.cfg
        return 2 * c.n_kv_heads * c.head_dim * 4 * (len(self.layers) - len(self._recurrent()))

    def step(self) -> None:
        so = lib.load()
        if self.world == 1:
            lib.check(so.tfb_qwen35_decode_step(C.byref(self.args), lib.stream()), "tfb_qwen35_decode_step")
            return
        part = lambda p, l=0: lib.check(so.tfb_qwen35_step_part(C.byref(self.args), p, l, lib.stream()), "tfb_qwen35_step_part")
        part(0)
        for l in range(len(self.layers)):
            part(1, l)                               # ... this rank's partial sums of the MoE block
            lib.check(so.tfb_moe_allreduce_finalize(C.byref(self._reduce_args), lib.stream()), "tfb_moe_allreduce_finalize")
        part(3)                                      # this rank's vocabulary slice -> (best logit, index)
        lib.check(so.tfb_pick_allgather(C.byref(self._pick_args), lib.stream()), "tfb_pick_allgather")
