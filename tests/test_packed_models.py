"""Weight preparation for MiniCPM3, granite and Qwen3.5: checkpoint keys -> authored names (alias tables) -> kernel
layout -> one file and back; a session built from the file decodes what a session built from the resource does."""
import pytest
import torch

from tilefoundry_b200.authored import granite_4_0_h_small as gr
from tilefoundry_b200.authored import minicpm3_4b as m
from tilefoundry_b200.authored import qwen3_5_35b_a3b as q35
from tilefoundry_b200.authored.weights import random_weights
from tilefoundry_b200.engine import packed_models as pm
from tilefoundry_b200.engine import sharding
from tilefoundry_b200.runtime import DictResource

BF = torch.bfloat16


def _minicpm3(seed=3):
    cfg = m.MINICPM3_TINY
    return cfg, m.tie_head(random_weights(m.build(cfg), seed=seed, std=0.05))


def _granite(seed=3):
    cfg = gr.GRANITE_TINY
    return cfg, random_weights(gr.build(cfg), seed=seed, std=0.05, overrides=gr.weight_overrides)


def _qwen35(seed=3):
    cfg = q35.QWEN3_5_TINY
    return cfg, random_weights(q35.build(cfg), seed=seed, std=0.05, overrides=q35.weight_overrides)


MODELS = {"minicpm3_4b": _minicpm3, "granite_4_0_h_small": _granite, "qwen3_5_35b_a3b": _qwen35}


def _minicpm3_state_dict(cfg, w):
    """The seeded authored weights under a Hugging Face MiniCPM3 checkpoint's keys and layouts (nn.Linear: (out, in))."""
    sd = {"model.embed_tokens.weight": w["w_embed"], "model.norm.weight": w["gamma_final"], "lm_head.weight": w["w_head"].t().contiguous()}
    norms = {"gamma_in": "input_layernorm.weight", "gamma_post": "post_attention_layernorm.weight",
             "gamma_q_a": "self_attn.q_a_layernorm.weight", "gamma_kv_a": "self_attn.kv_a_layernorm.weight"}
    proj = {"w_q_a": "self_attn.q_a_proj", "w_q_b": "self_attn.q_b_proj", "w_kv_a": "self_attn.kv_a_proj_with_mqa",
            "w_kv_b": "self_attn.kv_b_proj", "w_o": "self_attn.o_proj", "w_gate": "mlp.gate_proj", "w_up": "mlp.up_proj",
            "w_down": "mlp.down_proj"}
    for i in range(cfg.num_hidden_layers):
        for ours, theirs in norms.items():
            sd[f"model.layers.{i}.{theirs}"] = w[f"layer{i}.{ours}"]
        for ours, theirs in proj.items():
            sd[f"model.layers.{i}.{theirs}.weight"] = w[f"layer{i}.{ours}"][0].t().contiguous()
    return sd


def _granite_state_dict(cfg, w):
    """The seeded authored weights where a Hugging Face GraniteMoeHybrid checkpoint keeps them."""
    sd = {"model.embed_tokens.weight": w["table"], "model.norm.weight": w["gamma_final"]}
    mamba = {"w_in": "in_proj.weight", "conv_b": "conv1d.bias", "a_log": "A_log", "dt_bias": "dt_bias", "d_skip": "D",
             "gamma_ssm": "norm.weight", "w_out": "out_proj.weight"}
    attn = {"w_q": "q_proj.weight", "w_k": "k_proj.weight", "w_v": "v_proj.weight", "w_o": "o_proj.weight"}
    for i, kind in enumerate(cfg.layer_types):
        L, g = f"model.layers.{i}", lambda n: w[f"layer{i}.{n}"]
        if kind == "linear_attention":
            for ours, theirs in mamba.items():
                sd[f"{L}.mamba.{theirs}"] = g(f"mixer.{ours}")
            sd[f"{L}.mamba.conv1d.weight"] = g("mixer.conv_w").unsqueeze(1)
        else:
            for ours, theirs in attn.items():
                sd[f"{L}.self_attn.{theirs}"] = g(f"mixer.{ours}")
        sd[f"{L}.input_layernorm.weight"] = g("mixer.gamma_in")
        sd[f"{L}.post_attention_layernorm.weight"] = g("moe.gamma_post")
        sd[f"{L}.block_sparse_moe.input_linear.weight"] = torch.cat([g("moe.w_gate"), g("moe.w_up")], dim=1)
        sd[f"{L}.block_sparse_moe.output_linear.weight"] = g("moe.w_down")
        sd[f"{L}.block_sparse_moe.router.layer.weight"] = g("moe.router.w_router")
        sd[f"{L}.shared_mlp.input_linear.weight"] = g("moe.w_shared_in")
        sd[f"{L}.shared_mlp.output_linear.weight"] = g("moe.w_shared_out")
    return sd


def _same_packed(a, b):
    assert a.key == b.key and set(a.root) == set(b.root) and len(a.layers) == len(b.layers)
    for k in a.root:
        assert (a.root[k] is None) == (b.root[k] is None), k
        assert a.root[k] is None or torch.equal(a.root[k], b.root[k]), k
    for i, (x, y) in enumerate(zip(a.layers, b.layers)):
        assert set(x) == set(y), i
        for k in x:
            assert x[k].dtype == y[k].dtype and torch.equal(x[k], y[k]), (i, k)


def test_alias_tables_read_a_checkpoint_as_the_authored_weights():
    cfg, w = _minicpm3()
    _same_packed(pm.pack("minicpm3_4b", cfg, DictResource(_minicpm3_state_dict(cfg, w), alias=pm.hf_alias_minicpm3(cfg))),
                 pm.pack("minicpm3_4b", cfg, DictResource(w)))
    cfg, w = _granite()
    res = DictResource(_granite_state_dict(cfg, w), alias=pm.hf_alias_granite(cfg))
    for i, kind in enumerate(cfg.layer_types):                  # name by name, then the packed form
        sub = res.subtree(f"layer{i}")
        mixer = ("w_in", "conv_w", "conv_b", "a_log", "d_skip", "gamma_ssm", "w_out") if kind == "linear_attention" else ("w_q", "w_k", "w_v", "w_o")
        for n in mixer + ("gamma_in",):
            assert torch.equal(sub.subtree("mixer").load(n), w[f"layer{i}.mixer.{n}"]), (i, n)
        for n in ("gamma_post", "w_gate", "w_up", "w_down", "w_shared_in", "w_shared_out"):
            assert torch.equal(sub.subtree("moe").load(n), w[f"layer{i}.moe.{n}"]), (i, n)
        assert torch.equal(sub.subtree("moe").subtree("router").load("w_router"), w[f"layer{i}.moe.router.w_router"])
    _same_packed(pm.pack("granite_4_0_h_small", cfg, res), pm.pack("granite_4_0_h_small", cfg, DictResource(w)))


def _qwen35_state_dict(cfg, w, pre="model.language_model"):
    """A Hugging Face Qwen3.5-MoE checkpoint's keys and layouts holding the seeded weights: ``nn.Linear`` is (out, in),
    the experts' gate and up halves are one tensor, the norms store ``w`` of ``x * (1 + w)``.  Returns the state dict and
    the authored weights it stands for (the gains are what reading ``1 + w`` back gives)."""
    want = dict(w)
    lin = lambda t: t[0].t().contiguous()
    sd = {f"{pre}.embed_tokens.weight": w["table"], "lm_head.weight": w["w_head"].t().contiguous()}

    def gain(key, name):
        sd[key] = (w[name] - 1.0).to(BF)
        want[name] = sd[key].float() + 1.0
    gain(f"{pre}.norm.weight", "gamma_final")
    for i, kind in enumerate(cfg.layer_types):
        L, g = f"{pre}.layers.{i}", lambda n: w[f"layer{i}.{n}"]
        gain(f"{L}.input_layernorm.weight", f"layer{i}.mixer.gamma_in")
        gain(f"{L}.post_attention_layernorm.weight", f"layer{i}.moe.gamma_post")
        if kind == "linear_attention":
            for ours, theirs in (("w_in_qkv", "in_proj_qkv"), ("w_in_z", "in_proj_z"), ("w_in_b", "in_proj_b"),
                                 ("w_in_a", "in_proj_a"), ("w_out", "out_proj")):
                sd[f"{L}.linear_attn.{theirs}.weight"] = lin(g(f"mixer.{ours}"))
            sd[f"{L}.linear_attn.conv1d.weight"] = g("mixer.conv_w").unsqueeze(1)
            sd[f"{L}.linear_attn.A_log"], sd[f"{L}.linear_attn.dt_bias"] = g("mixer.a_log"), g("mixer.dt_bias")
            sd[f"{L}.linear_attn.norm.weight"] = g("mixer.gamma_gdn")
        else:
            for ours, theirs in (("w_qg", "q_proj"), ("w_k", "k_proj"), ("w_v", "v_proj"), ("w_o", "o_proj")):
                sd[f"{L}.self_attn.{theirs}.weight"] = lin(g(f"mixer.{ours}"))
            gain(f"{L}.self_attn.q_norm.weight", f"layer{i}.mixer.gamma_q")
            gain(f"{L}.self_attn.k_norm.weight", f"layer{i}.mixer.gamma_k")
        sd[f"{L}.mlp.experts.gate_up_proj"] = torch.cat([g("moe.w_gate"), g("moe.w_up")], dim=1)
        sd[f"{L}.mlp.experts.down_proj"] = g("moe.w_down")
        for ours, theirs in (("w_shared_gate", "shared_expert.gate_proj"), ("w_shared_up", "shared_expert.up_proj"),
                             ("w_shared_down", "shared_expert.down_proj"), ("w_shared_scale", "shared_expert_gate")):
            sd[f"{L}.mlp.{theirs}.weight"] = g(f"moe.{ours}").t().contiguous()
        sd[f"{L}.mlp.gate.weight"] = g("moe.router.w_router").t().contiguous()
    return sd, want


def test_qwen35_alias_table_applies_the_checkpoint_conversions():
    cfg, w = _qwen35()
    sd, want = _qwen35_state_dict(cfg, w)
    res = DictResource(sd, alias=pm.hf_alias_qwen3_5(cfg))
    for name, value in want.items():                             # name by name: value, shape and dtype as authored
        *path, leaf = name.split(".")
        sub = res
        for seg in path:
            sub = sub.subtree(seg)
        got = sub.load(leaf)
        assert got.dtype == value.dtype and got.shape == value.shape and torch.equal(got, value), name
    assert torch.equal(res.subtree("layer0").subtree("mixer").load("gamma_in"),
                       sd["model.language_model.layers.0.input_layernorm.weight"].float() + 1.0)
    _same_packed(pm.pack("qwen3_5_35b_a3b", cfg, res), pm.pack("qwen3_5_35b_a3b", cfg, DictResource(want)))
    # a tied head reads the embedding table
    tied = DictResource(sd, alias=pm.hf_alias_qwen3_5(cfg, head="model.language_model.embed_tokens.weight"))
    assert torch.equal(tied.load("w_head"), w["table"].t())


@pytest.mark.parametrize("key", sorted(MODELS))
def test_pack_save_load_round_trip(tmp_path, key):
    cfg, w = MODELS[key]()
    packed = pm.pack(key, cfg, DictResource(w))
    if key == "minicpm3_4b":
        assert packed.root["w_head"] is None                     # tied: the table is stored once
        assert packed.layers[0]["w_qkv_a"].shape == (cfg.q_lora_rank + cfg.kv_lora_rank + cfg.qk_rope_head_dim, cfg.hidden_size)
    path = tmp_path / f"{key}.safetensors"
    pm.save_packed(path, cfg, packed)
    _same_packed(pm.load_packed(path, key, cfg), packed)
    other = next(k for k in MODELS if k != key)
    with pytest.raises(ValueError, match="not a"):
        pm.load_packed(path, other, MODELS[other]()[0])
    import dataclasses
    field = "num_hidden_layers" if key != "qwen3_5_35b_a3b" else "vocab"
    with pytest.raises(ValueError, match=field):
        pm.load_packed(path, key, dataclasses.replace(cfg, **{field: getattr(cfg, field) + 8}))


def test_a_rank_cuts_its_shard_out_of_the_packed_layer():
    from tilefoundry_b200.engine import granite as ge
    from tilefoundry_b200.engine import qwen3_5 as qe
    cfg, w = _granite()
    layer = pm.pack("granite_4_0_h_small", cfg, DictResource(w)).layers[0]
    for rank in range(2):
        got = ge.shard_layer(layer, rank, 2)
        assert torch.equal(got["w_gate"], w["layer0.moe.w_gate"][rank::2]) and torch.equal(got["w_down"], w["layer0.moe.w_down"][rank::2])
        w_in, w_out = sharding.shared_slices(w["layer0.moe.w_shared_in"], w["layer0.moe.w_shared_out"], rank, 2)
        assert torch.equal(got["w_shared_in"], w_in) and torch.equal(got["w_shared_out"], w_out)
        assert got["w_in"] is layer["w_in"] and got["w_router"] is layer["w_router"]      # the mixer and router stay whole
    cfg, w = _qwen35()
    layer = pm.pack("qwen3_5_35b_a3b", cfg, DictResource(w)).layers[0]
    per = cfg.shared_intermediate // 2
    for rank in range(2):
        got = qe.shard_layer(cfg, layer, rank, 2)
        lo, hi = rank * per, (rank + 1) * per
        assert torch.equal(got["w_up"], w["layer0.moe.w_up"][rank::2])
        assert torch.equal(got["w_shared_gate"], qe._rows(w["layer0.moe.w_shared_gate"][..., lo:hi]))
        assert torch.equal(got["w_shared_down"], qe._rows(w["layer0.moe.w_shared_down"][..., lo:hi, :]))


@pytest.mark.gpu
@pytest.mark.parametrize("key", sorted(MODELS))
def test_session_from_packed_file_equals_session_from_resource(tmp_path, key):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tilefoundry_b200.engine.granite import GraniteSession
    from tilefoundry_b200.engine.minicpm3 import MiniCPM3Session
    from tilefoundry_b200.engine.qwen3_5 import Qwen35Session
    session = {"minicpm3_4b": MiniCPM3Session, "granite_4_0_h_small": GraniteSession, "qwen3_5_35b_a3b": Qwen35Session}[key]
    cfg, w = MODELS[key](seed=6)
    dev = torch.device("cuda:0")
    path = tmp_path / f"{key}.safetensors"
    pm.save_packed(path, cfg, pm.pack(key, cfg, DictResource(w)))
    vocab = cfg.vocab if key == "qwen3_5_35b_a3b" else cfg.vocab_size
    prompt = torch.randint(0, vocab, (20,), generator=torch.Generator().manual_seed(1))
    a = session(cfg, DictResource({k: v.to(dev) for k, v in w.items()}), max_ctx=128, device=dev)
    b = session(cfg, pm.load_packed(path, key, cfg, device=dev), max_ctx=128, device=dev)
    assert a.generate(prompt, 40).tokens == b.generate(prompt, 40).tokens
