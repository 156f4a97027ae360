"""Model, loss and objective against independent oracles: F.cross_entropy for the fused CE, and
(when the reference tree is mounted) the reference's own Qwen3 on CPU fp32 with shared weights."""

import os
import sys

import pytest
import torch
import torch.nn.functional as F

from tests.tiny import PARITY, TINY

# the reference package: an explicit checkout (TORCHURE_REFERENCE_DIR) or the offline install under baseline/_ref
_HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("TORCHURE_REFERENCE_DIR") or os.path.join(_HERE, "baseline", "_ref")


@pytest.mark.parametrize("shape", [(2, 128, 64, 1000, 64), (2, 256, 128, 5000, 512), (1, 100, 32, 300, 33)])
def test_fused_linear_ce_vs_cross_entropy(shape):
    from torchure_b200.loss import fused_linear_cross_entropy

    B, S, D, V, chunk = shape
    torch.manual_seed(0)
    h = torch.randn(B, S, D, requires_grad=True)
    w = (torch.randn(V, D) * 0.05).requires_grad_()
    y = torch.randint(0, V, (B, S))
    y[torch.rand(B, S) < 0.1] = -100
    loss = fused_linear_cross_entropy(h, w, y, -100, chunk)
    loss.backward()
    h2, w2 = h.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    ref = F.cross_entropy((h2 @ w2.t()).view(-1, V), y.view(-1), ignore_index=-100)
    ref.backward()
    torch.testing.assert_close(loss, ref, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(h.grad, h2.grad, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(w.grad, w2.grad, rtol=1e-4, atol=1e-6)
    with pytest.raises(RuntimeError):
        loss.backward()


def test_all_ignored_gives_zero():
    from torchure_b200.loss import fused_linear_cross_entropy

    h = torch.randn(4, 8, requires_grad=True)
    w = torch.randn(10, 8, requires_grad=True)
    loss = fused_linear_cross_entropy(h, w, torch.full((4,), -100), -100, 2)
    loss.backward()
    assert loss.item() == 0.0 and h.grad.abs().sum() == 0


def test_objective_fused_equals_plain():
    from torchure_b200.models import Qwen3
    from torchure_b200.objectives import ARObjective

    torch.manual_seed(0)
    m = Qwen3(**TINY)
    m.init_weights()
    ids = torch.randint(0, TINY["vocab_size"], (3, 16))
    batch = {"input_ids": ids, "labels": ids.clone()}
    a = ARObjective(fused_linear_ce=True, ce_chunk_size=7).compute_loss(m, batch)
    b = ARObjective(fused_linear_ce=False).compute_loss(m, batch)
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)


def test_param_order_and_count():
    from torchure_b200.models import Qwen3

    with torch.device("meta"):
        m = Qwen3(num_layers=28, num_heads=16, num_kv_heads=8, emb_dim=1024, head_dim=128, vocab_size=151936)
    assert m.num_params() == 574_029_824  # default ffn 2816
    with torch.device("meta"):
        m = Qwen3(num_layers=28, num_heads=16, num_kv_heads=8, emb_dim=1024, head_dim=128, vocab_size=151936,
                  ffn_dim=3072)
    assert m.num_params() == 596_049_920
    names = [n for n, _ in m.named_parameters()]
    assert names[0] == "token_emb.weight" and names[-1] == "norm.weight" and len(names) == 310
    assert names[1:12] == [f"blocks.0.{s}.weight" for s in (
        "gqa.q_proj", "gqa.k_proj", "gqa.v_proj", "gqa.o_proj", "gqa.q_norm", "gqa.k_norm", "norm1", "norm2",
        "ffn.gate_proj", "ffn.up_proj", "ffn.down_proj")]


def test_init_statistics():
    from torchure_b200.models import Qwen3

    torch.manual_seed(0)
    m = Qwen3(**PARITY)
    m.init_weights()
    L = PARITY["num_layers"]
    assert abs(m.blocks[0].gqa.q_proj.weight.std().item() - 0.02) < 2e-3
    assert abs(m.blocks[0].gqa.o_proj.weight.std().item() - 0.02 * (2 * L) ** -0.5) < 1e-3
    assert torch.equal(m.norm.weight, torch.ones_like(m.norm.weight))
    assert m.lm_head.weight is m.token_emb.weight


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "torchure")), reason="reference package not available")
def test_matches_reference_model_cpu_fp32():
    sys.path.insert(0, REF)
    try:
        from torchure.models.qwen3.qwen3 import Qwen3 as RefQwen3
    finally:
        sys.path.remove(REF)
    from torchure_b200.models import Qwen3

    cfg = dict(TINY)
    torch.manual_seed(0)
    ref = RefQwen3(**cfg)
    ref.init_weights()
    # the reference's norms use eps=None (fp32 machine epsilon)
    ours = Qwen3(**cfg, norm_eps=torch.finfo(torch.float32).eps)
    missing = ours.load_state_dict(ref.state_dict(), strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    ids = torch.randint(0, cfg["vocab_size"], (2, 16))
    torch.testing.assert_close(ours(ids), ref(ids), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(ours(ids, return_final_hidden=True), ref(ids, return_final_hidden=True),
                               rtol=1e-4, atol=1e-5)
    mask = torch.ones(2, 16, dtype=torch.long)
    mask[0, :5] = 0
    a, b = ours(ids, attention_mask=mask), ref(ids, attention_mask=mask)
    torch.testing.assert_close(a[mask.bool()], b[mask.bool()], rtol=1e-4, atol=1e-5)
    ours(ids).sum().backward()
    ref(ids).sum().backward()
    for (n, p), (_, q) in zip(ours.named_parameters(), ref.named_parameters()):
        torch.testing.assert_close(p.grad, q.grad, rtol=1e-3, atol=1e-5, msg=lambda m: f"{n}: {m}")


def _hf_pair(kind):
    """(our model, the Hugging Face implementation of the same architecture with our weights), tiny, fp32, CPU."""
    transformers = pytest.importorskip("transformers")
    from torchure_b200.models import Llama3, Qwen3

    torch.manual_seed(0)
    common = dict(num_layers=2, num_heads=4, num_kv_heads=2, emb_dim=64, vocab_size=97, ffn_dim=160)
    if kind == "llama3":
        ours = Llama3(**common)           # head_dim = emb / heads = 16, no QK-norm, theta 5e5, eps 1e-5
        hf_cfg = transformers.LlamaConfig(
            vocab_size=97, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=True,
            attention_bias=False, mlp_bias=False, max_position_embeddings=128)
        hf = transformers.LlamaForCausalLM(hf_cfg)
    else:
        ours = Qwen3(**common, head_dim=32)   # head_dim independent of emb / heads, QK-norm, theta 1e6, eps 1e-6
        hf_cfg = transformers.Qwen3Config(
            vocab_size=97, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=True,
            attention_bias=False, max_position_embeddings=128, use_sliding_window=False)
        hf = transformers.Qwen3ForCausalLM(hf_cfg)
    ours.init_weights()
    with torch.no_grad():
        for p in ours.parameters():   # non-trivial norm gains
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    sd = {"model.embed_tokens.weight": ours.token_emb.weight, "model.norm.weight": ours.norm.weight,
          "lm_head.weight": ours.lm_head.weight}
    for i, b in enumerate(ours.blocks):
        pre = f"model.layers.{i}."
        sd.update({pre + "self_attn.q_proj.weight": b.gqa.q_proj.weight, pre + "self_attn.k_proj.weight": b.gqa.k_proj.weight,
                   pre + "self_attn.v_proj.weight": b.gqa.v_proj.weight, pre + "self_attn.o_proj.weight": b.gqa.o_proj.weight,
                   pre + "mlp.gate_proj.weight": b.ffn.gate_proj.weight, pre + "mlp.up_proj.weight": b.ffn.up_proj.weight,
                   pre + "mlp.down_proj.weight": b.ffn.down_proj.weight, pre + "input_layernorm.weight": b.norm1.weight,
                   pre + "post_attention_layernorm.weight": b.norm2.weight})
        if kind != "llama3":
            sd[pre + "self_attn.q_norm.weight"] = b.gqa.q_norm.weight
            sd[pre + "self_attn.k_norm.weight"] = b.gqa.k_norm.weight
    missing, unexpected = hf.load_state_dict({k: v.detach().clone() for k, v in sd.items()}, strict=False)
    assert not unexpected and all("rotary" in m or "inv_freq" in m for m in missing), (missing, unexpected)
    return ours.eval(), hf.eval()


@pytest.mark.parametrize("kind", ["llama3", "qwen3"])
def test_models_match_the_hugging_face_implementations(kind):
    """Independent oracle for both model families: logits and input-embedding gradients of the Hugging Face
    implementation (random init, no download) loaded with our weights."""
    ours, hf = _hf_pair(kind)
    ids = torch.randint(0, 97, (2, 24), generator=torch.Generator().manual_seed(1))
    got = ours(ids)
    want = hf(input_ids=ids).logits
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    got.float().pow(2).mean().backward()
    want.float().pow(2).mean().backward()
    torch.testing.assert_close(ours.token_emb.weight.grad, hf.model.embed_tokens.weight.grad, rtol=1e-3, atol=1e-6)
    torch.testing.assert_close(ours.blocks[0].gqa.q_proj.weight.grad, hf.model.layers[0].self_attn.q_proj.weight.grad,
                               rtol=1e-3, atol=1e-6)


@pytest.mark.parametrize("kind", ["llama3", "qwen3"])
def test_hugging_face_round_trip(kind, tmp_path):
    """A Hugging Face directory (random init, written locally) imported into this layout gives the same logits;
    exported again it loads into the Hugging Face class with identical tensors."""
    transformers = pytest.importorskip("transformers")
    from torchure_b200.models import build_model
    from torchure_b200.models.hf import export_hf, import_hf

    _, hf = _hf_pair(kind)
    hf.save_pretrained(tmp_path / "hf_in")
    section = import_hf(str(tmp_path / "hf_in"), str(tmp_path / "model.pt"))
    assert section["name"] == ("llama3_2" if kind == "llama3" else "qwen3_dense")
    ours = build_model(section["name"], section["config"])
    ours.load_state_dict(torch.load(tmp_path / "model.pt"))
    ids = torch.randint(0, 97, (2, 24), generator=torch.Generator().manual_seed(2))
    torch.testing.assert_close(ours.eval()(ids), hf(input_ids=ids).logits, rtol=1e-4, atol=1e-5)
    export_hf(str(tmp_path / "model.pt"), section, str(tmp_path / "hf_out"))
    back = transformers.AutoModelForCausalLM.from_pretrained(tmp_path / "hf_out")
    for (n, a), (_, b) in zip(hf.state_dict().items(), back.state_dict().items()):
        assert torch.equal(a, b), n


def test_llama3_registry_and_defaults():
    from torchure_b200.models import build_model

    m = build_model("llama3_2", dict(num_layers=1, num_heads=4, num_kv_heads=2, emb_dim=64, vocab_size=50))
    assert m.cfg["head_dim"] == 16 and m.cfg["qk_norm"] is False and m.cfg["rope_theta"] == 500_000.0
    assert not hasattr(m.blocks[0].gqa, "q_norm")
    assert m.lm_head.weight is m.token_emb.weight
