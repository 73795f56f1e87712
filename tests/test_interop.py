"""Checkpoint interop on the CPU: a module tree shaped like a bitsandbytes-quantised, PEFT-wrapped Qwen2 model
(built from this repository's quantiser: bitsandbytes and peft are not installed) -> PackedLayers and LoRA
factors, and LoRA factors -> a PEFT adapter directory that reads back, header first, as the reference's
harness reads it (harness/run_task.py:62-72)."""

import math
from types import SimpleNamespace

import pytest
import torch

from decentrik_prime_b200 import interop, k_nf4, quantize
from oracle import nf4_oracle

H, KV, I = 256, 128, 512
SHAPES = {"q_proj": (H, H), "k_proj": (KV, H), "v_proj": (KV, H), "o_proj": (H, H),
          "gate_proj": (I, H), "up_proj": (I, H), "down_proj": (H, I)}


def fake_lora(base, seed, p=0.05):
    n, k = base.weight.quant_state.shape
    gen = torch.Generator().manual_seed(seed)
    A = SimpleNamespace(weight=(torch.rand(16, k, generator=gen) * 2 - 1) / math.sqrt(k), bias=None)
    B = SimpleNamespace(weight=torch.randn(n, 16, generator=gen) * 0.01, bias=None)
    return SimpleNamespace(base_layer=base, lora_A={"default": A}, lora_B={"default": B},
                           lora_dropout={"default": SimpleNamespace(p=p)}, scaling={"default": 2.0},
                           active_adapters=["default"], merged=False, disable_adapters=False)


def fake_model(n_layers=2, lora_on=("q_proj", "v_proj")):
    layers = []
    for i in range(n_layers):
        lin = {}
        for j, (name, (n, k)) in enumerate(SHAPES.items()):
            m = quantize.random_nf4_weight(n, k, seed=100 * i + j)
            m.bias = (torch.randn(n, generator=torch.Generator().manual_seed(j)) * 0.1).half().float() if name in ("q_proj", "k_proj", "v_proj") else None
            if m.bias is not None:
                m.bias = SimpleNamespace(data=m.bias)
            lin[name] = fake_lora(m, 1000 * i + j) if name in lora_on else m
        norm = lambda s: SimpleNamespace(weight=SimpleNamespace(data=torch.rand(H, generator=torch.Generator().manual_seed(s)) + 0.5),
                                         variance_epsilon=1e-6)
        layers.append(SimpleNamespace(self_attn=SimpleNamespace(**{n: lin[n] for n in interop.ATTN}),
                                      mlp=SimpleNamespace(**{n: lin[n] for n in interop.MLP}),
                                      input_layernorm=norm(7 + i), post_attention_layernorm=norm(9 + i)))
    qwen = SimpleNamespace(layers=layers)
    causal = SimpleNamespace(model=qwen)
    return SimpleNamespace(base_model=SimpleNamespace(model=causal))     # PeftModel -> LoraModel -> CausalLM -> Qwen2Model


def test_model_parts_repack_every_layer():
    model = fake_model()
    originals = []
    for layer in model.base_model.model.model.layers:
        w = {}
        for name in k_nf4.LAYER_WEIGHTS:
            mod = getattr(layer.self_attn if name in interop.ATTN else layer.mlp, name)
            base = getattr(mod, "base_layer", mod)
            st = base.weight.quant_state
            w[name] = nf4_oracle.dequant_ref(base.weight.data.numpy().copy(), st.absmax.numpy().copy(), st.state2.absmax.numpy().copy(),
                                             torch.full((st.state2.absmax.numel(),), float(st.offset)).numpy(), st.state2.code.numpy())
        originals.append(w)
    parts = interop.model_parts(model, "cpu")
    assert len(parts) == 2
    for p, orig in zip(parts, originals):
        assert set(p["lora"]) == {"q_proj", "v_proj"} and p["dropout"] == 0.05
        assert set(p["bias"]) == {"q_proj", "k_proj", "v_proj"}
        assert p["norm"][0].shape == (H,) and p["norm"][2] == 1e-6
        for name in k_nf4.LAYER_WEIGHTS:
            got = nf4_oracle.dequant_weight(p["layer"], name, p["code2"])
            assert tuple(got.shape) == SHAPES[name]
            assert torch.equal(got.reshape(-1), torch.from_numpy(orig[name]))
        A, B, scale = p["lora"]["q_proj"]
        assert A.shape == (16, H) and B.shape == (H, 16) and scale == 2.0


def test_unsupported_models_are_refused():
    model = fake_model(1)
    layer = model.base_model.model.model.layers[0]
    layer.self_attn.q_proj.merged = True
    with pytest.raises(interop.Unsupported):
        interop.model_parts(model, "cpu")
    layer.self_attn.q_proj.merged = False
    layer.self_attn.q_proj.lora_A["default"].weight = torch.zeros(8, H)          # rank 8
    layer.self_attn.q_proj.lora_B["default"].weight = torch.zeros(H, 8)
    with pytest.raises(interop.Unsupported):
        interop.model_parts(model, "cpu")
    model = fake_model(1)
    model.base_model.model.model.layers[0].mlp.up_proj = SimpleNamespace(weight=torch.zeros(I, H))      # not quantised
    with pytest.raises(interop.Unsupported):
        interop.model_parts(model, "cpu")


def test_adapter_directory_round_trip(tmp_path):
    parts = interop.model_parts(fake_model(3), "cpu")
    layers = [{n: (A, B) for n, (A, B, _) in p["lora"].items()} for p in parts]
    names = interop.save_adapter(tmp_path / "adapter", layers, alpha=32.0, dropout=0.05, base_model="Qwen/Qwen2.5-1.5B-Instruct")
    assert len(names) == 3 * 2 * 2
    header = interop.adapter_header(tmp_path / "adapter")
    assert header["base_model.model.model.layers.2.self_attn.v_proj.lora_B.weight"] == ["F32", [KV, 16]]
    assert header["base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight"] == ["F32", [16, H]]
    back, config = interop.load_adapter(tmp_path / "adapter")
    assert config["r"] == 16 and config["lora_alpha"] == 32.0 and config["target_modules"] == ["q_proj", "v_proj"]
    assert config["peft_type"] == "LORA" and config["lora_dropout"] == 0.05
    for a, b in zip(layers, back):
        for n in a:
            assert torch.equal(a[n][0], b[n][0]) and torch.equal(a[n][1], b[n][1])
    with pytest.raises(ValueError):
        interop.save_adapter(tmp_path / "bad", [{"q_proj": (torch.zeros(8, H), torch.zeros(H, 8))}])
