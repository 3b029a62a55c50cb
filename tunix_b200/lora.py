"""LoRA / QLoRA, in-tree.

The reference delegates adapters to an external library (`qwix`; tunix/cli/utils/model.py:31-77):
`LoraProvider(module_path=<regex>, rank, alpha[, weight_qtype="nf4", tile_size])` plus
`apply_lora_to_model(model, provider, **dummy_inputs)`. The same two names exist here.
What the rest of the framework assumes about adapters (and what this module guarantees):

* adapter tensors are separate parameters named `<linear>.lora_a` ([r, in]) / `<linear>.lora_b` ([out, r]);
* only they are trainable, optimised, checkpointed and synced to the sampler
  (tunix/sft/peft_trainer.py:340-342, tunix/sft/checkpoint_manager.py:247-250, tunix/rl/rl_cluster.py:1288-1294);
* the frozen backbone can be shared between actor and reference: `disable_adapters(model)` gives the
  reference policy without a second copy of the weights (tunix/rl/rl_cluster.py:220-223);
* the effective weight is `W + (B @ A) * alpha / r` (tunix/models/safetensors_saver.py:106).
"""
from __future__ import annotations

import contextlib
import dataclasses
import math
import re
from typing import Iterator, Optional

import torch
import torch.nn as nn

from .models.transformer import Linear

# The 16 quantiles of a standard normal used by 4-bit NormalFloat.
_NF4_CODE = [-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
             -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
             0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
             0.7229568362236023, 1.0]


@dataclasses.dataclass
class LoraProvider:
    module_path: str = r".*(q_proj|k_proj|v_proj|o_proj|gate_proj|up_proj|down_proj)"
    rank: int = 8
    alpha: float = 16.0
    weight_qtype: Optional[str] = None   # "nf4" -> QLoRA
    tile_size: int = 64                  # quantisation block size
    dropout: float = 0.0


_DEQUANT_SCRATCH: dict = {}      # (shape, device) -> bf16 tensor, see NF4Weight.dequantize(shared=True)


class NF4Weight:
    """Block-wise 4-bit NormalFloat storage of a frozen weight: two codes per byte + fp32 absmax per block."""

    def __init__(self, w: torch.Tensor, block: int = 64):
        self.shape, self.dtype, self.block = tuple(w.shape), w.dtype, block
        flat = w.detach().float().reshape(-1)
        pad = (-flat.numel()) % block
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        blocks = flat.view(-1, block)
        self.absmax = blocks.abs().amax(dim=1).clamp_min(1e-12)
        normed = blocks / self.absmax[:, None]
        code = torch.tensor(_NF4_CODE, device=w.device)
        idx = (normed.unsqueeze(-1) - code).abs().argmin(dim=-1).to(torch.uint8).view(-1)
        self.packed = (idx[0::2] << 4) | idx[1::2]
        self.numel = w.numel()

    def dequantize(self, shared: bool = False) -> torch.Tensor:
        """The bf16 (or original dtype) weight. `shared`: write into a scratch tensor that every NF4 weight of this
        shape on this device reuses: valid until the next such call, for consumers that run on the same stream
        right away (a projection's GEMMs); the expanded weight then never outlives the layer that uses it."""
        if self.packed.is_cuda and self.dtype == torch.bfloat16:
            # one kernel: codebook lookup, block scale, bf16 store (csrc/optim.cu)
            from . import _lib
            _lib.register_cuda_sigs({"tb_nf4_dequant": [_lib.P, _lib.P, _lib.I, _lib.P, _lib.LL, _lib.P]})
            if self.packed.numel() % 8:
                self.packed = torch.cat([self.packed, self.packed.new_zeros(8 - self.packed.numel() % 8)])
            if shared:
                key = (self.shape, self.packed.device)
                out = _DEQUANT_SCRATCH.get(key)
                if out is None:
                    out = _DEQUANT_SCRATCH[key] = torch.empty(self.shape, dtype=torch.bfloat16, device=self.packed.device)
            else:
                out = torch.empty(self.shape, dtype=torch.bfloat16, device=self.packed.device)
            rc = _lib.cuda().tb_nf4_dequant(self.packed.data_ptr(), self.absmax.data_ptr(), self.block, out.data_ptr(),
                                            self.numel, _lib.stream_ptr())
            _lib.check(rc, "tb_nf4_dequant")
            return out
        code = torch.tensor(_NF4_CODE, device=self.packed.device)
        idx = torch.stack([(self.packed >> 4) & 0xF, self.packed & 0xF], dim=1).view(-1).long()
        vals = code[idx].view(-1, self.block) * self.absmax[:, None]
        return vals.view(-1)[: self.numel].view(self.shape).to(self.dtype)

    def to(self, device):
        self.packed, self.absmax = self.packed.to(device), self.absmax.to(device)
        return self


def _matches(provider: LoraProvider, name: str) -> bool:
    return re.fullmatch(provider.module_path, name) is not None or re.search(provider.module_path, name) is not None


def apply_lora_to_model(model: nn.Module, provider: LoraProvider, seed: int = 0, **_unused_model_inputs) -> nn.Module:
    """Attach adapters to every `Linear` whose dotted name matches `provider.module_path`; freeze the rest."""
    gen = torch.Generator().manual_seed(seed)
    n_wrapped = 0
    for name, mod in model.named_modules():
        if not isinstance(mod, Linear) or not _matches(provider, name):
            continue
        dev, dt = mod.weight.device, mod.weight.dtype
        a = torch.empty(provider.rank, mod.in_features)
        # Kaiming-uniform A, zero B: the adapted model starts identical to the base model.
        bound = 1.0 / math.sqrt(mod.in_features)
        a.uniform_(-bound, bound, generator=gen)
        out_rows = mod.out_features
        tp = getattr(mod, "tp", None)
        if tp is not None and tp.world > 1:
            # the projection was sliced for tensor parallelism: the adapter factor on the split side is sliced with it
            # (the full A is drawn first, so the adapted model is the same for every tp size)
            if mod.tp_mode == "row":
                n = mod.in_features // tp.world
                a = a[:, tp.rank * n:(tp.rank + 1) * n].contiguous()
            else:
                out_rows = mod.out_features // tp.world
        mod.lora_a = nn.Parameter(a.to(device=dev, dtype=dt))
        mod.lora_b = nn.Parameter(torch.zeros(out_rows, provider.rank, device=dev, dtype=dt))
        if tp is not None and tp.world > 1:
            sliced = mod.lora_a if mod.tp_mode == "row" else mod.lora_b
            sliced.shard_spec, sliced.shard_group = ((1 if mod.tp_mode == "row" else 0), tp.rank, tp.world), tp.group
        mod.lora_scale = provider.alpha / provider.rank
        if provider.weight_qtype == "nf4":
            mod.quant = NF4Weight(mod.weight.data, provider.tile_size)
            mod.weight.data = torch.empty(0, device=dev, dtype=dt)  # drop the dense copy
        n_wrapped += 1
    if n_wrapped == 0:
        raise ValueError(f"no module matched LoRA pattern {provider.module_path!r}")
    for pname, p in model.named_parameters():
        p.requires_grad_(is_lora_param_name(pname))
    if getattr(model, "tp", None) is not None:
        from .parallel.tp import mark_sharded_params
        mark_sharded_params(model)
    model._lora_provider = provider
    return model


def is_lora_param_name(name: str) -> bool:
    return name.endswith("lora_a") or name.endswith("lora_b")


def is_lora_enabled(model: nn.Module) -> bool:
    """True if the model carries adapter parameters (tunix/sft/utils.py:75-79)."""
    return any(is_lora_param_name(n) for n, _ in model.named_parameters())


def lora_parameters(model: nn.Module) -> Iterator[tuple[str, nn.Parameter]]:
    for n, p in model.named_parameters():
        if is_lora_param_name(n):
            yield n, p


def lora_state_dict(model: nn.Module) -> dict:
    return {n: p.detach() for n, p in lora_parameters(model)}


@contextlib.contextmanager
def disable_adapters(model: nn.Module):
    """Run the frozen backbone (the reference policy) through the same module tree."""
    mods = [m for m in model.modules() if isinstance(m, Linear) and m.lora_a is not None]
    prev = [m.lora_enabled for m in mods]
    for m in mods:
        m.lora_enabled = False
    try:
        yield model
    finally:
        for m, p in zip(mods, prev):
            m.lora_enabled = p


@torch.no_grad()
def merged_weight(mod: Linear) -> torch.Tensor:
    """W + (B @ A) * alpha / r in the base dtype."""
    w = mod.base_weight()
    if mod.lora_a is None:
        return w
    return (w.float() + (mod.lora_b.float() @ mod.lora_a.float()) * mod.lora_scale).to(w.dtype)


@torch.no_grad()
def merge_lora_(model: nn.Module) -> nn.Module:
    """Fold adapters into the base weights and remove them."""
    for mod in model.modules():
        if isinstance(mod, Linear) and mod.lora_a is not None:
            w = merged_weight(mod)
            mod.quant = None
            mod.weight.data = w
            mod.lora_a = mod.lora_b = None
    return model
