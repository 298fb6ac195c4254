"""Weight preparation: checkpoint keys -> authored names (alias table) -> kernel layout -> one file and back."""
import pytest
import torch

from tilefoundry_b200.authored import qwen3_1_7b as q
from tilefoundry_b200.authored.weights import random_weights
from tilefoundry_b200.engine import packed
from tilefoundry_b200.runtime import DictResource

BF = torch.bfloat16


def _hf_state_dict(cfg, weights):
    """The seeded authored weights under a Hugging Face checkpoint's keys and layouts (nn.Linear: (out, in))."""
    sd = {"model.embed_tokens.weight": weights["w_embed"], "model.norm.weight": weights["gamma_final"]}
    norms = {"gamma_in": "input_layernorm.weight", "gamma_post": "post_attention_layernorm.weight",
             "gamma_q": "self_attn.q_norm.weight", "gamma_k": "self_attn.k_norm.weight"}
    proj = {"w_q": "self_attn.q_proj", "w_k": "self_attn.k_proj", "w_v": "self_attn.v_proj", "w_o": "self_attn.o_proj",
            "w_gate": "mlp.gate_proj", "w_up": "mlp.up_proj", "w_down": "mlp.down_proj"}
    for i in range(cfg.num_hidden_layers):
        for ours, theirs in norms.items():
            sd[f"model.layers.{i}.{theirs}"] = weights[f"layer{i}.{ours}"]
        for ours, theirs in proj.items():
            sd[f"model.layers.{i}.{theirs}.weight"] = weights[f"layer{i}.{ours}"][0].t().contiguous()
    return sd


def test_alias_table_reads_a_checkpoint_as_the_authored_weights():
    cfg = q.QWEN3_TINY
    weights = q.tie_head(random_weights(q.build(cfg), seed=3, std=0.05))
    res = DictResource(_hf_state_dict(cfg, weights), alias=packed.hf_alias(cfg))
    assert torch.equal(res.load("w_embed"), weights["w_embed"])
    assert torch.equal(res.load("w_head"), weights["w_head"])
    for i in range(cfg.num_hidden_layers):
        sub = res.subtree(f"layer{i}")
        for name in ("gamma_in", "gamma_q", "w_q", "w_k", "w_v", "w_o", "w_gate", "w_up", "w_down"):
            got = sub.load(name)
            assert got.shape == weights[f"layer{i}.{name}"].shape and torch.equal(got, weights[f"layer{i}.{name}"]), name


def test_pack_save_load_round_trip(tmp_path):
    cfg = q.QWEN3_TINY
    weights = q.tie_head(random_weights(q.build(cfg), seed=4, std=0.05))
    from_authored = packed.pack(cfg, DictResource(weights))
    from_checkpoint = packed.pack(cfg, DictResource(_hf_state_dict(cfg, weights), alias=packed.hf_alias(cfg)))
    assert from_authored.root["w_head"] is None                       # tied: the table is stored once
    H, I = cfg.hidden_size, cfg.intermediate_size
    QP, KVP = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    for a, b, i in zip(from_authored.layers, from_checkpoint.layers, range(cfg.num_hidden_layers)):
        assert a["w_qkv"].shape == (QP + 2 * KVP, H) and a["w_gate_up"].shape == (2 * I, H) and a["w_down"].shape == (H, I)
        assert torch.equal(a["w_qkv"][:QP], weights[f"layer{i}.w_q"][0].t())
        assert torch.equal(a["w_gate_up"][I:], weights[f"layer{i}.w_up"][0].t())
        assert a["w_gate"].data_ptr() == a["w_gate_up"].data_ptr()     # views, not copies
        for k in packed.LAYER_TENSORS:
            assert torch.equal(a[k], b[k]), k
    path = tmp_path / "tiny.safetensors"
    packed.save_packed(path, cfg, from_authored)
    back = packed.load_packed(path, cfg)
    assert back.root["w_head"] is None and torch.equal(back.root["w_embed"], from_authored.root["w_embed"])
    for a, b in zip(from_authored.layers, back.layers):
        for k in packed.LAYER_TENSORS + ("w_gate", "w_up"):
            assert a[k].dtype == b[k].dtype == BF and torch.equal(a[k], b[k]), k
    other = q.Qwen3Config(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                          intermediate_size=512, vocab_size=1024, num_hidden_layers=2, max_position_embeddings=512)
    with pytest.raises(ValueError, match="num_hidden_layers"):
        packed.load_packed(path, other)


@pytest.mark.gpu
def test_session_from_packed_file_equals_session_from_resource(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tilefoundry_b200.engine.qwen3 import Qwen3Session
    cfg, dev = q.QWEN3_TINY, torch.device("cuda:0")
    weights = q.tie_head(random_weights(q.build(cfg), seed=6, std=0.05))
    path = tmp_path / "tiny.safetensors"
    packed.save_packed(path, cfg, packed.pack(cfg, DictResource(weights)))
    prompt = torch.randint(0, cfg.vocab_size, (20,), generator=torch.Generator().manual_seed(1))
    a = Qwen3Session(cfg, DictResource({k: v.to(dev) for k, v in weights.items()}), max_ctx=128, device=dev)
    b = Qwen3Session(cfg, packed.load_packed(path, cfg, device=dev), max_ctx=128, device=dev)
    assert a.generate(prompt, 50).tokens == b.generate(prompt, 50).tokens
    assert b.w_head.data_ptr() == b.w_embed.data_ptr()
