"""Gemma 4 text decoder (tunix/models/gemma4/model.py, attention.py, layers.py, moe.py, config.py:149-464).

What sets it apart from Gemma 3, and how each piece runs here:

* per-layer inputs: a second embedding table `[V, L * Dp]` plus a projection of the token embedding give every
  layer its own `Dp`-wide input, gated into the residual stream after the feed-forward block;
* local (sliding-window) layers use `head_dim`, global layers `global_head_dim` (512) with partial rotary
  (the first `global_rope_proportion` of the frequency pairs rotate, the rest stay put) and, with
  `k_eq_v_global`, fewer kv heads and values that are the un-normalised key projection;
* keys, queries are RMS-normalised with a scale, values without; the softmax scale is 1;
* the last `num_kv_shared_layers` layers have no k/v projections: they attend over the keys and values of the last
  earlier layer of the same attention type (in training: that layer's tensors of the same forward pass; with a
  KV cache: that layer's cache), and may use a double-wide MLP;
* optional MoE block next to the dense MLP: a router on the RMS-normalised residual (scale vector, 1/sqrt(D),
  softmax, top-k, renormalise, per-expert scale), GeGLU experts, and separate post-norms for both branches;
* every layer's output is multiplied by a stored scalar; logits are soft-capped.

Attention with head_dim 64 / 128 / 256 runs on the tcgen05 flash kernels; the 512-wide global heads fall to the
PyTorch reference attention (`ops.reference.attention_ref`), the projections, norms, GLU and experts use the same
CUDA ops as the other families. Vision and audio encoders are not part of this module.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
from torch import nn

from ..ops import functional as F
from .config import ModelConfig, RematConfig
from .transformer import MLP, Linear, RMSNorm, Transformer, _GradBoundary, _torch_checkpoint


@dataclass
class Gemma4Config(ModelConfig):
    global_head_dim: int = 512
    num_global_kv_heads: Optional[int] = None     # kv heads of global layers when k_eq_v_global
    k_eq_v_global: bool = False
    global_rope_proportion: float = 0.25
    num_kv_shared_layers: int = 0
    kv_shared_hidden_dim: Optional[int] = None    # MLP width of the kv-sharing layers (E2B: twice hidden_dim)
    per_layer_input_dim: int = 0
    vocab_size_per_layer_input: Optional[int] = None

    def __post_init__(self):
        if self.layer_type(self.num_layers - 1) != "global":
            # the last layer always attends globally
            pat = [self.layer_type(i) for i in range(self.num_layers)]
            pat[-1] = "global"
            self.layer_pattern = tuple(pat)

    @property
    def first_kv_shared_layer(self) -> int:
        return self.num_layers - self.num_kv_shared_layers

    def kv_source(self, i: int) -> Optional[int]:
        """Layer whose keys / values layer i reuses (None: it has its own)."""
        first = self.first_kv_shared_layer
        if self.num_kv_shared_layers <= 0 or i < first:
            return None
        kind = self.layer_type(i)
        for j in range(first - 1, -1, -1):
            if self.layer_type(j) == kind:
                return j
        raise ValueError(f"no unshared {kind} layer before layer {i}")

    def kv_shape(self, i: int):
        """(kv heads, head dim) of layer i."""
        if self.layer_type(i) == "local":
            return self.num_kv_heads, self.head_dim
        kh = self.num_global_kv_heads if (self.k_eq_v_global and self.num_global_kv_heads) else self.num_kv_heads
        return kh, (self.global_head_dim or self.head_dim)

    # ------------------------------------------------------------------ presets (config.py:235-414)
    @classmethod
    def _base(cls, **kw):
        base = dict(family="gemma4", vocab_size=262144, head_dim=256, rope_theta=1_000_000.0, local_rope_theta=10_000.0,
                    norm_eps=1e-6, weight_tying=True, qk_norm=True, norm_add_one=False, embed_scale=True, activation="gelu",
                    final_logit_softcap=30.0, post_norms=True, max_position=131072,
                    layer_pattern=("local",) * 5 + ("global",))
        base.update(kw)
        return cls(**base)

    @classmethod
    def gemma4_e2b(cls):
        return cls._base(num_layers=35, embed_dim=1536, hidden_dim=6144, num_heads=8, num_kv_heads=1, sliding_window=512,
                         per_layer_input_dim=256, num_kv_shared_layers=20, kv_shared_hidden_dim=12288,
                         layer_pattern=("local",) * 4 + ("global",))

    @classmethod
    def gemma4_e4b(cls):
        return cls._base(num_layers=42, embed_dim=2560, hidden_dim=10240, num_heads=8, num_kv_heads=2, sliding_window=512,
                         per_layer_input_dim=256, num_kv_shared_layers=18)

    @classmethod
    def gemma4_12b(cls):
        return cls._base(num_layers=48, embed_dim=3840, hidden_dim=15360, num_heads=16, num_kv_heads=8,
                         num_global_kv_heads=1, k_eq_v_global=True, sliding_window=1024)

    @classmethod
    def gemma4_31b(cls):
        return cls._base(num_layers=60, embed_dim=5376, hidden_dim=21504, num_heads=32, num_kv_heads=16,
                         num_global_kv_heads=4, k_eq_v_global=True, sliding_window=1024)

    @classmethod
    def gemma4_26b_a4b(cls):
        return cls._base(num_layers=30, embed_dim=2816, hidden_dim=2112, num_heads=16, num_kv_heads=8,
                         num_global_kv_heads=2, k_eq_v_global=True, sliding_window=1024, num_experts=128,
                         num_experts_per_tok=8, moe_hidden_dim=704)


def _rope_tables(cfg: Gemma4Config, local: bool, device):
    """cos / sin [max_position, H/2]; global layers rotate only the first `global_rope_proportion` of the pairs
    (the remaining inverse frequencies are zero: cos 1, sin 0)."""
    H = cfg.head_dim if local else (cfg.global_head_dim or cfg.head_dim)
    half = H // 2
    theta = cfg.local_rope_theta if (local and cfg.local_rope_theta) else cfg.rope_theta
    rot = half if local else int(cfg.global_rope_proportion * H // 2)
    inv = torch.zeros(half, dtype=torch.float64, device=device)
    inv[:rot] = 1.0 / (theta ** (torch.arange(0, rot, dtype=torch.float64, device=device) * 2.0 / H))
    ang = torch.arange(cfg.max_position, dtype=torch.float64, device=device)[:, None] * inv[None, :]
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


class Gemma4Attention(nn.Module):
    def __init__(self, cfg: Gemma4Config, layer_idx: int, device=None):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.is_local = cfg.layer_type(layer_idx) == "local"
        self.window = cfg.sliding_window if self.is_local else 0
        self.kv_heads, self.H = cfg.kv_shape(layer_idx)
        self.kv_source = cfg.kv_source(layer_idx)
        self.scale = 1.0
        D, N, H, dt = cfg.embed_dim, cfg.num_heads, self.H, cfg.dtype
        self.q_proj = Linear(D, N * H, False, dt, device)
        self.o_proj = Linear(N * H, D, False, dt, device)
        self.q_norm = RMSNorm(H, cfg.norm_eps, False, dt, device)
        self.k_proj = self.v_proj = self.k_norm = None
        if self.kv_source is None:
            self.k_proj = Linear(D, self.kv_heads * H, False, dt, device)
            if not (cfg.k_eq_v_global and not self.is_local):
                self.v_proj = Linear(D, self.kv_heads * H, False, dt, device)
            self.k_norm = RMSNorm(H, cfg.norm_eps, False, dt, device)
        self.register_buffer("_unit", torch.ones(H, dtype=dt, device=device), persistent=False)

    def forward(self, x, positions, rope, cache=None, segment_ids=None, attention_mask=None, shared=None):
        """Returns (attention output before the post-norm, new cache entry, what a kv-sharing layer needs)."""
        cfg = self.cfg
        B, T, _ = x.shape
        N, KH, H = cfg.num_heads, self.kv_heads, self.H
        cos, sin = rope
        q = F.rope(self.q_norm(self.q_proj(x).view(B, T, N, H)), positions, cos, sin)
        new_cache = None
        if self.kv_source is None:
            k = self.k_proj(x).view(B, T, KH, H)
            v = self.v_proj(x).view(B, T, KH, H) if self.v_proj is not None else k
            k = F.rope(self.k_norm(k), positions, cos, sin)
            v = F.rmsnorm(v, self._unit, cfg.norm_eps, False)
            seg_q = seg_k = segment_ids
            q_off = None
            if cache is not None:
                ck, cv, cseg, end = cache["k"], cache["v"], cache["seg"], cache["end"]
                ck[:, end:end + T] = k.detach()
                cv[:, end:end + T] = v.detach()
                cseg[:, end:end + T] = segment_ids.to(cseg.dtype) if segment_ids is not None else 1
                new_end = end + T
                k, v, seg_k = ck[:, :new_end], cv[:, :new_end], cseg[:, :new_end]
                seg_q, q_off = seg_k[:, end:new_end], end
                new_cache = {"k": ck, "v": cv, "seg": cseg, "end": new_end}
            shared = (k, v, seg_q, seg_k, q_off)
        else:
            if shared is None:
                raise RuntimeError(f"layer {self.layer_idx} shares the keys / values of layer {self.kv_source}")
            k, v, seg_q, seg_k, q_off = shared
            if cache is not None:
                new_cache = {"end": cache["end"] + T}
        if attention_mask is not None:
            from ..ops import reference as R
            o = R.attention_ref(q, k, v, scale=self.scale, softcap=0.0,
                                mask=attention_mask[:, None] if attention_mask.dim() == 3 else attention_mask)
        else:
            o = F.attention(q, k, v, scale=self.scale, causal=True, window=self.window, softcap=0.0, q_off=q_off,
                            seg_q=seg_q, seg_k=seg_k)
        return self.o_proj(o.reshape(B, T, N * H)), new_cache, shared


class Gemma4MoE(nn.Module):
    """Router + GeGLU experts of the MoE checkpoints (tunix/models/gemma4/moe.py:80-217). The expert weights are
    stacked `[E, F, D]` (gate, up) and `[E, D, F]` (down), the layout the grouped GEMMs take."""

    def __init__(self, cfg: Gemma4Config, device=None):
        super().__init__()
        E, D, Fd, dt = cfg.num_experts, cfg.embed_dim, cfg.moe_hidden_dim, cfg.dtype
        self.cfg = cfg
        self.router = Linear(D, E, False, dt, device)
        self.router_scale = nn.Parameter(torch.ones(D, dtype=dt, device=device))
        self.per_expert_scale = nn.Parameter(torch.ones(E, dtype=dt, device=device))
        self.gate_proj = nn.Parameter(torch.empty(E, Fd, D, dtype=dt, device=device))
        self.up_proj = nn.Parameter(torch.empty(E, Fd, D, dtype=dt, device=device))
        self.down_proj = nn.Parameter(torch.empty(E, D, Fd, dtype=dt, device=device))
        self.register_buffer("_unit", torch.ones(D, dtype=dt, device=device), persistent=False)
        self.ep = None
        self.ep_group = None
        self.last_routed_experts = None
        self.last_aux_loss = None

    def route(self, xt):
        cfg = self.cfg
        h = F.rmsnorm(xt, self._unit, cfg.norm_eps, False)
        h = h * self.router_scale * (cfg.embed_dim ** -0.5)
        probs = torch.softmax(self.router(h).float(), dim=-1)
        w, idx = torch.topk(probs, cfg.num_experts_per_tok, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        return w * self.per_expert_scale.float()[idx], idx

    def forward(self, routed_from, expert_in):
        """routed_from [T, D]: what the router sees (the residual stream); expert_in [T, D]: its pre-normed copy."""
        from ..parallel import moe_dispatch
        w, idx = self.route(routed_from)
        self.last_routed_experts = idx
        return moe_dispatch.expert_forward(self, expert_in, w.to(expert_in.dtype), idx)


class Gemma4DecoderLayer(nn.Module):
    def __init__(self, cfg: Gemma4Config, layer_idx: int, device=None):
        super().__init__()
        dt, D = cfg.dtype, cfg.embed_dim
        mk = lambda: RMSNorm(D, cfg.norm_eps, False, dt, device)  # noqa: E731
        self.cfg = cfg
        self.self_attn = Gemma4Attention(cfg, layer_idx, device)
        shared = cfg.kv_source(layer_idx) is not None
        width = cfg.kv_shared_hidden_dim if (shared and cfg.kv_shared_hidden_dim) else cfg.hidden_dim
        self.mlp = MLP(cfg.replace(hidden_dim=width), device)
        self.input_layernorm, self.post_attention_layernorm = mk(), mk()
        self.pre_feedforward_layernorm, self.post_feedforward_layernorm = mk(), mk()
        self.register_buffer("layer_scalar", torch.ones(1, dtype=dt, device=device))
        self.moe = None
        if cfg.num_experts > 0:
            self.moe = Gemma4MoE(cfg, device)
            self.post_feedforward_layernorm_1, self.post_feedforward_layernorm_2 = mk(), mk()
            self.pre_feedforward_layernorm_2 = mk()
        if cfg.per_layer_input_dim:
            Dp = cfg.per_layer_input_dim
            self.per_layer_input_gate = Linear(D, Dp, False, dt, device)
            self.per_layer_projection = Linear(Dp, D, False, dt, device)
            self.post_per_layer_input_norm = mk()

    def forward(self, x, positions, rope, cache=None, segment_ids=None, attention_mask=None, shared=None,
                per_layer_input=None):
        cfg = self.cfg
        a, new_cache, shared = self.self_attn(self.input_layernorm(x), positions, rope, cache, segment_ids, attention_mask,
                                              shared)
        x = x + self.post_attention_layernorm(a)
        m = self.mlp(self.pre_feedforward_layernorm(x))
        if self.moe is not None:
            flat = x.reshape(-1, x.shape[-1])
            e = self.moe(flat, self.pre_feedforward_layernorm_2(flat)).view_as(x)
            m = self.post_feedforward_layernorm_1(m) + self.post_feedforward_layernorm_2(e)
        x = x + self.post_feedforward_layernorm(m)
        if cfg.per_layer_input_dim:
            g = torch.nn.functional.gelu(self.per_layer_input_gate(x), approximate="tanh") * per_layer_input
            x = x + self.post_per_layer_input_norm(self.per_layer_projection(g))
        return x * self.layer_scalar, new_cache, shared


class Gemma4Transformer(Transformer):
    """Same call interface as `Transformer` (tokens, positions, dense KV cache, segment ids, skip_lm_head), so
    the trainers, the dense `Sampler` and the log-prob helpers work unchanged."""

    def __init__(self, cfg: Gemma4Config, device=None):
        nn.Module.__init__(self)
        self.config = cfg
        self.layer_grad_hook = None
        dt, D, L = cfg.dtype, cfg.embed_dim, cfg.num_layers
        self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, D, dtype=dt, device=device))
        self.layers = nn.ModuleList([Gemma4DecoderLayer(cfg, i, device) for i in range(L)])
        self.norm = RMSNorm(D, cfg.norm_eps, False, dt, device)
        self.lm_head = None if cfg.weight_tying else nn.Parameter(torch.empty(cfg.vocab_size, D, dtype=dt, device=device))
        if cfg.per_layer_input_dim:
            Dp = cfg.per_layer_input_dim
            Vp = cfg.vocab_size_per_layer_input or cfg.vocab_size
            self.embed_tokens_per_layer = nn.Parameter(torch.empty(Vp, L * Dp, dtype=dt, device=device))
            self.per_layer_model_projection = Linear(D, L * Dp, False, dt, device)
            self.per_layer_projection_norm = RMSNorm(Dp, cfg.norm_eps, False, dt, device)
        self._rope_cache = {}
        self.tp = None

    def _rope(self, local: bool, device):
        key = (local, str(device))
        tab = self._rope_cache.get(key)
        if tab is None:
            tab = self._rope_cache[key] = _rope_tables(self.config, local, device)
        return tab

    def per_layer_inputs(self, tokens, x):
        """[B, T, L, Dp]: (norm(projection of the token embedding) + per-layer embedding) / sqrt(2)."""
        cfg = self.config
        B, T = tokens.shape
        L, Dp = cfg.num_layers, cfg.per_layer_input_dim
        e = F.embedding(tokens, self.embed_tokens_per_layer, math.sqrt(Dp)).view(B, T, L, Dp)
        p = (self.per_layer_model_projection(x) * (cfg.embed_dim ** -0.5)).view(B, T, L, Dp)
        return (self.per_layer_projection_norm(p) + e) * (2.0 ** -0.5)

    def forward(self, input_tokens, positions=None, cache=None, attention_mask=None, segment_ids=None,
                skip_lm_head: bool = False, output_hidden_states: bool = False):
        cfg = self.config
        x = F.embedding(input_tokens, self.embed_tokens, math.sqrt(cfg.embed_dim))
        ple = self.per_layer_inputs(input_tokens, x) if cfg.per_layer_input_dim else None
        return self.forward_embeddings(x, positions=positions, cache=cache, attention_mask=attention_mask,
                                       segment_ids=segment_ids, skip_lm_head=skip_lm_head,
                                       output_hidden_states=output_hidden_states, per_layer_inputs=ple)

    def forward_embeddings(self, x, positions=None, cache=None, attention_mask=None, segment_ids=None,
                           skip_lm_head: bool = False, output_hidden_states: bool = False, batch_shape=None,
                           per_layer_inputs=None):
        cfg = self.config
        B, T = x.shape[:2]
        dev = x.device
        if cfg.per_layer_input_dim and per_layer_inputs is None:
            raise ValueError("this checkpoint needs per-layer inputs; call forward() with token ids")
        if positions is None:
            start = 0 if cache is None else cache[0]["end"]
            positions = torch.arange(start, start + T, device=dev, dtype=torch.int32)[None].expand(B, T)
        positions = positions.to(torch.int32).contiguous()
        new_cache = [] if cache is not None else None
        use_remat = cfg.remat_config != RematConfig.NONE and torch.is_grad_enabled() and cache is None
        hook = self.layer_grad_hook if (torch.is_grad_enabled() and cache is None) else None
        kv = {}                          # layer index -> keys / values for the layers that share them
        sources = {cfg.kv_source(i) for i in range(cfg.num_layers)} - {None}
        for i, layer in enumerate(self.layers):
            rope = self._rope(cfg.layer_type(i) == "local", dev)
            if hook is not None and x.requires_grad:
                x = _GradBoundary.apply(x, i, hook)
            ple = per_layer_inputs[:, :, i] if per_layer_inputs is not None else None
            src = cfg.kv_source(i)
            args = (x, positions, rope, None if cache is None else cache[i], segment_ids, attention_mask,
                    kv.get(src) if src is not None else None, ple)
            if use_remat:
                x, c, shared = _torch_checkpoint(layer, *args, use_reentrant=False)
            else:
                x, c, shared = layer(*args)
            if i in sources:
                kv[i] = shared
            if new_cache is not None:
                new_cache.append(c)
        if hook is not None and x.requires_grad:
            x = _GradBoundary.apply(x, len(self.layers), hook)
        x = self.norm(x)
        if skip_lm_head or output_hidden_states:
            return x, new_cache
        return self.compute_final_logits(x), new_cache

    def init_cache(self, batch_size: int, cache_size: int, dtype=None, device=None):
        cfg = self.config
        dtype = dtype or cfg.dtype
        device = device or self.embed_tokens.device
        out = []
        for i in range(cfg.num_layers):
            if cfg.kv_source(i) is not None:
                out.append({"end": 0})              # attends over the cache of its source layer
                continue
            kh, h = cfg.kv_shape(i)
            mk = lambda: torch.zeros(batch_size, cache_size, kh, h, dtype=dtype, device=device)  # noqa: E731
            out.append({"k": mk(), "v": mk(), "seg": torch.zeros(batch_size, cache_size, dtype=torch.int32, device=device),
                        "end": 0})
        return out

    def aux_loss(self):
        return None


def create_gemma4(cfg: Gemma4Config, device=None, seed: int = 0, init: bool = True) -> Gemma4Transformer:
    model = Gemma4Transformer(cfg, device=device)
    if init:
        model.init_weights(seed)        # matrices only: norm scales, router scales and layer scalars stay at one
    return model
