"""Checkpoint interop: decoder layers of a bitsandbytes-quantised, PEFT-wrapped Qwen2 model -> PackedLayers and
LoRA factors for this library, and LoRA factors -> a PEFT adapter directory.

Loading follows what the reference's runner checks and collects when it takes a model over
(solution/fast_qwen.py:65-93 `_lora_parts`, 96-97 `_is_bnb_4bit`, 180-216 the per-layer walk) and repacks with
the same routine (solution/k_nf4.py:126-173 through k_nf4.repack_layer). Everything is duck-typed, as in the
reference: bitsandbytes and peft themselves are not imported (neither is installed where this library is
built), any module tree with the same attribute names works, and the tests build one from this repository's
own quantiser.

Saving writes what PEFT's `save_pretrained` leaves on disk and what the reference's harness reads back
(harness/run_task.py:62-72 reads tensor names, shapes and dtypes from the safetensors header;
harness/check_rules.py:171-182 compares adapter_config.json): `adapter_model.safetensors` with
`base_model.model.model.layers.{i}.{self_attn|mlp}.{proj}.lora_{A|B}.weight` in fp32 and an
`adapter_config.json`.
"""

import json
import os
import struct

import torch

from . import k_nf4

ATTN = ("q_proj", "k_proj", "v_proj", "o_proj")
MLP = ("gate_proj", "up_proj", "down_proj")


class Unsupported(ValueError):
    """The model uses something this path does not implement (the reference raises the same kind of error and
    falls back to the stock trainer, solution/fast_qwen.py:55-63)."""


def _require(cond, msg):
    if not cond:
        raise Unsupported(msg)


def is_4bit_linear(module):
    """A bitsandbytes 4-bit linear, recognised the way the reference does (solution/fast_qwen.py:96-97), or
    anything that quacks like one (a `.weight` with a `.quant_state`)."""
    w = getattr(module, "weight", None)
    return w is not None and hasattr(w, "quant_state")


def lora_parts(module, adapter="default"):
    """(A fp32 [r,K], B fp32 [N,r], dropout p, scaling) of a PEFT LoRA layer, checked to be plain LoRA
    (reference solution/fast_qwen.py:65-93)."""
    for attr in ("lora_A", "lora_B", "lora_dropout", "scaling", "base_layer"):
        _require(hasattr(module, attr), f"{type(module).__name__} is not a PEFT LoRA layer")
    active = getattr(module, "active_adapters", [adapter])
    _require(list(active) == [adapter], "exactly one active adapter expected")
    _require(not getattr(module, "merged", False), "merged adapter")
    _require(not getattr(module, "disable_adapters", False), "adapters disabled")
    for flag, what in (("use_dora", "DoRA"), ("lora_bias", "LoRA bias")):
        v = getattr(module, flag, {})
        _require(not (v.get(adapter, False) if isinstance(v, dict) else v), what)
    _require(adapter not in getattr(module, "lora_variant", {}), "LoRA variant")
    a, b = module.lora_A[adapter], module.lora_B[adapter]
    _require(getattr(a, "bias", None) is None and getattr(b, "bias", None) is None, "LoRA A/B with bias")
    drop = module.lora_dropout[adapter]
    p = float(getattr(drop, "p", 0.0))
    _require(a.weight.dtype == torch.float32 and b.weight.dtype == torch.float32, "LoRA weights are expected in fp32")
    return a.weight, b.weight, p, float(module.scaling[adapter])


def layer_parts(layer, device, adapter="default"):
    """One decoder layer (attributes self_attn.{q,k,v,o}_proj, mlp.{gate,up,down}_proj, input_layernorm,
    post_attention_layernorm) as what stack.DecoderLayerProjections(parts=...) takes:
    {"layer": PackedLayer on `device`, "code2", "bias": {name: fp16}, "lora": {name: (A, B, scale)},
     "dropout": p, "norm": (w_in fp32, w_post fp32, eps)}.
    A projection may be a plain 4-bit linear or a PEFT LoRA wrapper around one."""
    device = torch.device(device)
    mods = {name: getattr(layer.self_attn, name) for name in ATTN}
    mods.update({name: getattr(layer.mlp, name) for name in MLP})
    linears, lora, p_seen = {}, {}, set()
    for name, mod in mods.items():
        base = mod
        if hasattr(mod, "lora_A"):
            A, B, p, scaling = lora_parts(mod, adapter)
            _require(A.shape[0] == 16 and B.shape[1] == 16, f"{name}: LoRA rank {A.shape[0]} (the kernels implement 16)")
            lora[name] = (A, B, scaling)
            p_seen.add(p)
            base = mod.base_layer
        _require(is_4bit_linear(base), f"{name} is not a 4-bit linear")
        linears[name] = base
    _require(len(p_seen) <= 1, "one LoRA dropout probability expected")
    try:
        packed, code2 = k_nf4.repack_layer(linears, device)
    except ValueError as exc:
        raise Unsupported(str(exc)) from exc
    bias = {}
    for name, mod in linears.items():
        b = getattr(mod, "bias", None)
        if b is not None:
            b16 = b.data.to(device, torch.float16)
            _require(torch.equal(b16.float(), b.data.to(device).float()), f"{name} bias not fp16-representable")
            bias[name] = b16
    norm = None
    if hasattr(layer, "input_layernorm") and hasattr(layer, "post_attention_layernorm"):
        eps = float(getattr(layer.input_layernorm, "variance_epsilon", 1e-6))
        norm = (layer.input_layernorm.weight.data.to(device).float().contiguous(),
                layer.post_attention_layernorm.weight.data.to(device).float().contiguous(), eps)
    return {"layer": packed, "code2": code2, "bias": bias, "lora": lora, "dropout": p_seen.pop() if p_seen else 0.0,
            "norm": norm}


def model_parts(model, device, adapter="default"):
    """layer_parts of every decoder layer of a (possibly PEFT-wrapped) causal LM: the layer list is looked up
    as the reference does (peft_model.base_model.model.model.layers, solution/fast_qwen.py:132-140)."""
    node = model
    for _ in range(4):                       # PeftModel -> LoraModel -> Qwen2ForCausalLM -> Qwen2Model
        if hasattr(node, "layers"):
            break
        node = getattr(node, "base_model", None) or getattr(node, "model", None)
        _require(node is not None, "no decoder layers found")
    _require(hasattr(node, "layers"), "no decoder layers found")
    parts = [layer_parts(layer, device, adapter) for layer in node.layers]
    code = parts[0]["code2"]
    _require(all(torch.equal(p["code2"], code) for p in parts), "second-level code tables differ between layers")
    return parts


# --------------------------------------------------------------------------------------------------------
# PEFT adapter directory
# --------------------------------------------------------------------------------------------------------
def _module_path(i, name):
    return f"base_model.model.model.layers.{i}.{'self_attn' if name in ATTN else 'mlp'}.{name}"


def save_adapter(directory, layers, alpha=32.0, dropout=0.05, base_model="", rank=16):
    """Write `adapter_model.safetensors` + `adapter_config.json` into `directory`.
    `layers`: one dict per decoder layer, projection name -> (A [r,K], B [N,r]) (any float dtype; saved as
    fp32, which is what the reference's adapters hold, solution/fast_qwen.py:89-90)."""
    from safetensors.torch import save_file
    os.makedirs(directory, exist_ok=True)
    tensors, targets = {}, set()
    for i, layer in enumerate(layers):
        for name, (A, B) in layer.items():
            if A.shape[0] != rank or B.shape[1] != rank:
                raise ValueError(f"layer {i} {name}: rank {A.shape[0]} / {B.shape[1]}, expected {rank}")
            tensors[_module_path(i, name) + ".lora_A.weight"] = A.detach().to("cpu", torch.float32).contiguous()
            tensors[_module_path(i, name) + ".lora_B.weight"] = B.detach().to("cpu", torch.float32).contiguous()
            targets.add(name)
    save_file(tensors, os.path.join(directory, "adapter_model.safetensors"), metadata={"format": "pt"})
    config = {"peft_type": "LORA", "task_type": "CAUSAL_LM", "base_model_name_or_path": base_model, "r": rank,
              "lora_alpha": alpha, "lora_dropout": dropout, "target_modules": sorted(targets), "bias": "none",
              "fan_in_fan_out": False, "inference_mode": True, "init_lora_weights": True, "use_dora": False,
              "use_rslora": False, "modules_to_save": None, "layers_to_transform": None, "layers_pattern": None,
              "rank_pattern": {}, "alpha_pattern": {}, "revision": None}
    with open(os.path.join(directory, "adapter_config.json"), "w", encoding="utf-8") as fh:
        json.dump(config, fh, indent=2, sort_keys=True)
    return sorted(tensors)


def adapter_header(directory):
    """{tensor name: [dtype, shape]} read from the safetensors header alone, as the reference's harness does
    (harness/run_task.py:62-72)."""
    with open(os.path.join(directory, "adapter_model.safetensors"), "rb") as fh:
        size = struct.unpack("<Q", fh.read(8))[0]
        header = json.loads(fh.read(size))
    return {name: [info.get("dtype"), info.get("shape")] for name, info in sorted(header.items()) if name != "__metadata__"}


def load_adapter(directory, device="cpu"):
    """(layers, config): the inverse of save_adapter."""
    from safetensors.torch import load_file
    tensors = load_file(os.path.join(directory, "adapter_model.safetensors"), device=str(device))
    with open(os.path.join(directory, "adapter_config.json"), encoding="utf-8") as fh:
        config = json.load(fh)
    layers = {}
    for key, t in tensors.items():
        parts = key.split(".")
        i, name, which = int(parts[parts.index("layers") + 1]), parts[-3], parts[-2]
        slot = layers.setdefault(i, {}).setdefault(name, [None, None])
        slot[0 if which == "lora_A" else 1] = t
    return [{n: tuple(ab) for n, ab in layers[i].items()} for i in sorted(layers)], config


def stack_adapter(stack):
    """The LoRA masters of a stack.ProjectionStack as save_adapter's `layers` argument."""
    return [{name: (p.A, p.B) for name, p in layer.proj.items() if p.has_lora} for layer in stack._distinct]
