"""Generic pre-norm decoder covering Llama 3.x, Qwen2.5, Qwen3 (dense + MoE), Gemma 1/2/3 (text).

Model contract (the one every trainer / sampler in this package relies on; it mirrors
tunix/models/qwen3/model.py:1359-1463):

    logits_or_hidden, cache = model(input_tokens, positions=None, cache=None, attention_mask=None,
                                    segment_ids=None, skip_lm_head=False, output_hidden_states=False)
    model.compute_final_logits(hidden)            # fp32 logits, final soft-cap applied
    model.token_logprobs(hidden, targets, ...)    # fused lm_head -> log-softmax -> gather
    model.init_cache(batch, cache_size, dtype)    # dense KV cache for the vanilla sampler
    model.get_model_input()                       # dummy inputs (LoRA tracing helper in the reference)

Weights keep the HF `[out, in]` layout, so safetensors import/export is a rename.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint as _torch_checkpoint

from ..ops import functional as F
from ..ops import reference as R
from .config import ModelConfig, RematConfig


class _JointRowsFn(torch.autograd.Function):
    """Parameters that lie back to back in one storage, seen as one tensor without a copy; the gradient of the joint
    tensor is handed back as row slices."""

    @staticmethod
    def forward(ctx, joint, *parts):
        ctx.rows = [p.shape[0] for p in parts]
        ctx.set_materialize_grads(False)
        return joint.view_as(joint)

    @staticmethod
    def backward(ctx, g):
        if g is None:                  # the consumer added the gradient into the joint `main_grad` itself
            return (None,) * (1 + len(ctx.rows))
        return (None, *g.split(ctx.rows, 0))


def _joint_rows(parts):
    """cat(parts, 0) for tensors of equal trailing shape: a view when they already follow each other in memory (the
    optimizers' flat parameter buffers lay q / k / v weights out that way), a copy otherwise."""
    first = parts[0]
    off, adjacent = first.storage_offset(), all(p.is_contiguous() for p in parts)
    for p in parts:
        if not adjacent or p.untyped_storage().data_ptr() != first.untyped_storage().data_ptr() or p.storage_offset() != off \
                or p.shape[1:] != first.shape[1:]:
            adjacent = False
            break
        off += p.numel()
    if not adjacent:
        return torch.cat(list(parts), 0)
    rows = sum(p.shape[0] for p in parts)
    joint = first.detach().as_strided((rows, *first.shape[1:]), first.stride(), first.storage_offset())
    if torch.is_grad_enabled() and any(p.requires_grad for p in parts):
        out = _JointRowsFn.apply(joint, *parts)
        mgs = [getattr(p, "main_grad", None) for p in parts]
        if all(m is not None for m in mgs):
            # gradient slots that follow each other as well: consumers accumulate straight into the joint slot
            m0, moff, ok = mgs[0], mgs[0].storage_offset(), True
            for m, p_ in zip(mgs, parts):
                ok = ok and m.is_contiguous() and m.untyped_storage().data_ptr() == m0.untyped_storage().data_ptr() \
                    and m.storage_offset() == moff and m.shape == p_.shape
                moff += m.numel()
            if ok:
                out.main_grad = m0.as_strided((rows, *m0.shape[1:]), m0.stride(), m0.storage_offset())
                out._joint_parts = list(parts)
        return out
    return joint


class Linear(nn.Module):
    """Linear layer with optional bias, LoRA adapters and NF4-quantised frozen base (QLoRA)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, dtype=torch.float32, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        self.lora_a: Optional[nn.Parameter] = None
        self.lora_b: Optional[nn.Parameter] = None
        self.lora_scale = 0.0
        self.lora_enabled = True
        self.quant = None  # set by lora.quantize_base_nf4

    def base_weight(self) -> torch.Tensor:
        if self.quant is not None:
            return self.quant.dequantize()
        return self.weight

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        comm = getattr(self, "dp_shard", None)
        if comm is not None:
            # the weight is this rank's block of rows; the GEMM gathers the rest from the peers as it runs
            from ..parallel import fsdp3
            y = fsdp3.sharded_linear(x, self.weight, self.bias, None if self.lora_a is not None else residual, comm)
            if self.lora_a is not None and self.lora_enabled:
                y = F.lora_delta(x, self.lora_a, self.lora_b, y, self.lora_scale)
                return y if residual is None else y + residual
            return y
        if self.lora_a is not None and self.lora_enabled:
            # a quantised base is expanded inside the function (forward and again in backward) into a scratch that
            # all layers share, so no expanded weight is kept for the backward pass
            w = self.weight if self.quant is None else None
            return F.lora_linear(x, w, self.bias, self.lora_a, self.lora_b, self.lora_scale, residual, quant=self.quant)
        if self.quant is not None:
            keeps = torch.is_grad_enabled() and x.requires_grad          # autograd would hold on to the scratch
            return F.linear(x, self.quant.dequantize(shared=not keeps), self.bias, residual)
        return F.linear(x, self.weight, self.bias, residual)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, add_one: bool, dtype=torch.float32, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device) if add_one
                                   else torch.ones(dim, dtype=dtype, device=device))
        self.eps, self.add_one = eps, add_one

    def forward(self, x):
        return F.rmsnorm(x, self.weight, self.eps, self.add_one)


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device=None):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        D, N, K, H = cfg.embed_dim, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        dt = cfg.dtype
        self.q_proj = Linear(D, N * H, cfg.qkv_bias, dt, device)
        self.k_proj = Linear(D, K * H, cfg.qkv_bias, dt, device)
        self.v_proj = Linear(D, K * H, cfg.qkv_bias, dt, device)
        self.o_proj = Linear(N * H, D, False, dt, device)
        if cfg.qk_norm:
            self.q_norm = RMSNorm(H, cfg.norm_eps, cfg.norm_add_one, dt, device)
            self.k_norm = RMSNorm(H, cfg.norm_eps, cfg.norm_add_one, dt, device)
        self.is_local = cfg.layer_type(layer_idx) == "local"
        self.window = cfg.sliding_window if self.is_local else 0
        qpas = cfg.query_pre_attn_scalar if cfg.query_pre_attn_scalar else float(H)
        self.scale = 1.0 / math.sqrt(qpas)

    def forward(self, x, positions, rope, cache=None, segment_ids=None, attention_mask=None, residual=None):
        cfg = self.cfg
        B, T, _ = x.shape
        N, K, H = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        tp = getattr(self.q_proj, "tp", None)
        if tp is not None:
            # sequence-parallel input [B/tp, T, D]: one all-gather feeds q, k and v of this rank's heads
            from ..parallel import tp as tp_lib
            projs = (self.q_proj, self.k_proj, self.v_proj)
            if cache is not None:
                raise NotImplementedError("tensor parallelism covers training without a KV cache")
            self._tp_plain = not any(p.lora_a is not None or p.quant is not None for p in projs + (self.o_proj,))
            if self._tp_plain:
                w = _joint_rows([p.weight for p in projs])
                b = _joint_rows([p.bias for p in projs]) if self.q_proj.bias is not None else None
                qkv = tp_lib.column_parallel_linear(x, w, b, tp)
                B, N, K = qkv.shape[0], N // tp.world, K // tp.world
                q, k, v = qkv.split([N * H, K * H, K * H], dim=-1)
                q, k, v = (t.contiguous().view(B, T, -1, H) for t in (q, k, v))
            else:
                # adapters or a quantised base: gather the tokens once, then this rank's slices run as local projections
                xg = tp_lib.gather_tokens(x, tp)
                B, N, K = xg.shape[0], N // tp.world, K // tp.world
                q = self.q_proj(xg).view(B, T, N, H)
                k = self.k_proj(xg).view(B, T, K, H)
                v = self.v_proj(xg).view(B, T, K, H)
        else:
            q = self.q_proj(x).view(B, T, N, H)
            k = self.k_proj(x).view(B, T, K, H)
            v = self.v_proj(x).view(B, T, K, H)
        if cfg.qk_norm:
            q = self.q_norm(q)
            k = self.k_norm(k)
        cos, sin = rope
        q = F.rope(q, positions, cos, sin)
        k = F.rope(k, positions, cos, sin)
        seg_q = seg_k = segment_ids
        q_off = None
        new_cache = None
        if cache is not None:
            # dense cache [B,S,K,H]; this call writes positions [end, end+T)
            ck, cv, cseg, end = cache["k"], cache["v"], cache["seg"], cache["end"]
            ck[:, end:end + T] = k.detach()
            cv[:, end:end + T] = v.detach()
            if segment_ids is not None:
                cseg[:, end:end + T] = segment_ids.to(cseg.dtype)
            else:
                cseg[:, end:end + T] = 1
            new_end = end + T
            k, v = ck[:, :new_end], cv[:, :new_end]
            seg_k = cseg[:, :new_end]
            seg_q = seg_k[:, end:new_end]
            q_off = end
            new_cache = {"k": ck, "v": cv, "seg": cseg, "end": new_end}
        cp = getattr(self, "cp", None)
        if cp is not None and cp.world > 1:
            # context parallel: x holds this rank's tokens; keys and values of all earlier tokens come from the group
            if cache is not None or attention_mask is not None:
                raise NotImplementedError("context parallelism covers training without a KV cache or dense mask")
            k, v, seg_k, q_off = cp.keys_for_local_queries(k, v, segment_ids)
        if attention_mask is not None:
            o = R.attention_ref(q, k, v, scale=self.scale, softcap=cfg.attn_logit_softcap,
                                mask=attention_mask[:, None] if attention_mask.dim() == 3 else attention_mask)
        else:
            o = F.attention(q, k, v, scale=self.scale, causal=True, window=self.window,
                            softcap=cfg.attn_logit_softcap, q_off=q_off, seg_q=seg_q, seg_k=seg_k)
        o = o.reshape(B, T, N * H)
        if tp is not None:
            if self._tp_plain:
                return tp_lib.row_parallel_linear(o, self.o_proj.weight, residual, tp), new_cache
            y = tp_lib.scatter_sum_tokens(self.o_proj(o), tp)
            return (y if residual is None else y + residual), new_cache
        return self.o_proj(o, residual=residual), new_cache


class MLP(nn.Module):
    def __init__(self, cfg: ModelConfig, device=None):
        super().__init__()
        D, Fd, dt = cfg.embed_dim, cfg.hidden_dim, cfg.dtype
        self.gate_proj = Linear(D, Fd, False, dt, device)
        self.up_proj = Linear(D, Fd, False, dt, device)
        self.down_proj = Linear(Fd, D, False, dt, device)
        self.kind = cfg.activation

    def forward(self, x, residual=None):
        tp = getattr(self.gate_proj, "tp", None)
        if tp is not None:
            from ..parallel import tp as tp_lib
            if any(p.lora_a is not None or p.quant is not None for p in (self.gate_proj, self.up_proj, self.down_proj)):
                xg = tp_lib.gather_tokens(x, tp)
                h = F.glu(self.gate_proj(xg), self.up_proj(xg), self.kind)
                y = tp_lib.scatter_sum_tokens(self.down_proj(h), tp)
                return y if residual is None else y + residual
            gu = tp_lib.column_parallel_linear(x, torch.cat([self.gate_proj.weight, self.up_proj.weight], 0), None, tp)
            g, u = gu.split(gu.shape[-1] // 2, dim=-1)
            h = F.glu(g.contiguous(), u.contiguous(), self.kind)
            return tp_lib.row_parallel_linear(h, self.down_proj.weight, residual, tp)
        h = F.glu(self.gate_proj(x), self.up_proj(x), self.kind)
        return self.down_proj(h, residual=residual)


class MoELayer(nn.Module):
    """Top-k softmax-routed experts with SwiGLU (tunix/models/qwen3/model.py:851-1149).

    Router: softmax over experts -> top-k -> renormalise. Expert weights are stacked
    `[E, F, D]` (gate, up) and `[E, D, F]` (down). The optional auxiliary load-balancing loss
    (Switch-style: E * sum_e f_e * P_e) is stored in `self.last_aux_loss`.
    """

    def __init__(self, cfg: ModelConfig, device=None):
        super().__init__()
        E, D, Fd, dt = cfg.num_experts, cfg.embed_dim, cfg.moe_hidden_dim, cfg.dtype
        self.cfg = cfg
        self.router = Linear(D, E, False, dt, device)
        self.gate_proj = nn.Parameter(torch.empty(E, Fd, D, dtype=dt, device=device))
        self.up_proj = nn.Parameter(torch.empty(E, Fd, D, dtype=dt, device=device))
        self.down_proj = nn.Parameter(torch.empty(E, D, Fd, dtype=dt, device=device))
        self.last_aux_loss: Optional[torch.Tensor] = None
        self.last_routed_experts: Optional[torch.Tensor] = None
        self.ep = None        # parallel.ep.EPContext once shard_experts has kept this rank's experts
        self.ep_group = None

    def forward(self, x, residual=None, forced_experts: Optional[torch.Tensor] = None, recompute_experts: bool = False):
        cfg = self.cfg
        B, T, D = x.shape
        E, k = cfg.num_experts, cfg.num_experts_per_tok
        xt = x.reshape(B * T, D)
        logits = self.router(xt).float()
        w, idx, probs = R.topk_router_ref(logits, k, cfg.norm_topk_prob)
        if forced_experts is not None:  # router replay: reuse the sampler's expert choice
            fe = forced_experts.reshape(B * T, k).long()
            use = (fe >= 0).all(-1, keepdim=True)
            idx = torch.where(use, fe.clamp(min=0), idx)
            w_forced = probs.gather(1, idx)
            w = w_forced / w_forced.sum(-1, keepdim=True) if cfg.norm_topk_prob else w_forced
        self.last_routed_experts = idx.view(B, T, k)
        if cfg.router_aux_loss_coef > 0:
            frac = torch.zeros(E, device=x.device, dtype=torch.float32)
            frac.scatter_add_(0, idx.reshape(-1), torch.ones(idx.numel(), device=x.device))
            frac = frac / max(idx.numel(), 1)
            self.last_aux_loss = cfg.router_aux_loss_coef * E * (frac * probs.mean(0)).sum()
        from ..parallel import moe_dispatch
        y = moe_dispatch.expert_forward(self, xt, w, idx, recompute=recompute_experts)
        y = y.view(B, T, D)
        return y if residual is None else y + residual


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device=None):
        super().__init__()
        dt = cfg.dtype
        mk = lambda: RMSNorm(cfg.embed_dim, cfg.norm_eps, cfg.norm_add_one, dt, device)  # noqa: E731
        self.cfg = cfg
        self.input_layernorm = mk()
        self.self_attn = Attention(cfg, layer_idx, device)
        self.post_attention_layernorm = mk()
        self.mlp = MoELayer(cfg, device) if cfg.is_moe else MLP(cfg, device)
        if cfg.post_norms:
            self.post_attn_norm = mk()   # Gemma-2/3: norm on the attention output before the residual add
            self.post_ffw_norm = mk()

    def forward(self, x, positions, rope, cache=None, segment_ids=None, attention_mask=None, forced_experts=None):
        cfg = self.cfg
        h = self.input_layernorm(x)
        kw = {"forced_experts": forced_experts} if (forced_experts is not None and cfg.is_moe) else {}
        if cfg.post_norms:
            a, new_cache = self.self_attn(h, positions, rope, cache, segment_ids, attention_mask)
            x = x + self.post_attn_norm(a)
            m = self.mlp(self.post_attention_layernorm(x), **kw)
            x = x + self.post_ffw_norm(m)
        else:
            x, new_cache = self.self_attn(h, positions, rope, cache, segment_ids, attention_mask, residual=x)
            x = self.mlp(self.post_attention_layernorm(x), residual=x, **kw)
        return x, new_cache


def _moe_layer_split_remat(layer: DecoderLayer, x, positions, rope, segment_ids, attention_mask, forced):
    """Activation recomputation for an expert-parallel MoE layer that does not repeat the token exchange: the
    attention half (norm, projections, attention, second norm) is recomputed in backward as usual, the expert block
    keeps the rows it received and rebuilds only its own activations (`ops.moe.local_experts(recompute=True)`).
    Recomputing the whole layer instead would run dispatch and combine, both all-to-all exchanges with their
    barriers, a second time in every backward pass."""
    def attn_half(x_):
        h = layer.input_layernorm(x_)
        x1, _ = layer.self_attn(h, positions, rope, None, segment_ids, attention_mask, residual=x_)
        return x1, layer.post_attention_layernorm(x1)
    x1, h2 = _torch_checkpoint(attn_half, x, use_reentrant=False)
    return layer.mlp(h2, residual=x1, forced_experts=forced, recompute_experts=True)


class _GradBoundary(torch.autograd.Function):
    """Identity whose backward tells a listener that backward has passed this point of the network."""

    @staticmethod
    def forward(ctx, x, idx, hook):
        ctx.idx, ctx.hook = idx, hook
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.hook(ctx.idx)
        return g, None, None


class Transformer(nn.Module):
    def __init__(self, cfg: ModelConfig, device=None):
        super().__init__()
        self.config = cfg
        self.layer_grad_hook = None  # callable(int): backward reached the input of layer i (L = after last layer)
        dt = cfg.dtype
        self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, cfg.embed_dim, dtype=dt, device=device))
        self.layers = nn.ModuleList([DecoderLayer(cfg, i, device) for i in range(cfg.num_layers)])
        self.norm = RMSNorm(cfg.embed_dim, cfg.norm_eps, cfg.norm_add_one, dt, device)
        self.lm_head = None if cfg.weight_tying else nn.Parameter(
            torch.empty(cfg.vocab_size, cfg.embed_dim, dtype=dt, device=device))
        self._rope_cache: dict = {}
        self.tp = None  # parallel.tp.TPContext once apply_tensor_parallel has sliced the weights
        self.cp = None  # parallel.cp.ContextParallel once apply_context_parallel has split the sequence axis

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02) -> "Transformer":
        """Random normal(0, std) for matrices, identity scale for norms, zero biases and LoRA-B."""
        dev = self.embed_tokens.device
        gen = torch.Generator(device=dev).manual_seed(seed)
        for name, p in self.named_parameters():
            if p.dim() >= 2 and "lora_b" not in name:
                if p.numel() > (1 << 28):  # fill huge tensors in slices to bound temporaries
                    flat = p.view(-1)
                    step = 1 << 26
                    for s0 in range(0, flat.numel(), step):
                        flat[s0:s0 + step].normal_(0.0, std, generator=gen)
                else:
                    p.normal_(0.0, std, generator=gen)
            elif "lora_b" in name or name.endswith("bias"):
                p.zero_()
        return self

    def head_weight(self) -> torch.Tensor:
        return self.embed_tokens if self.lm_head is None else self.lm_head

    def _rope(self, local: bool, device):
        cfg = self.config
        key = (local, str(device))
        tab = self._rope_cache.get(key)
        if tab is None:
            theta = cfg.local_rope_theta if (local and cfg.local_rope_theta) else cfg.rope_theta
            sf = 1.0 if local else cfg.rope_scale_factor
            tab = R.rope_tables(cfg.head_dim, cfg.max_position, theta, sf, device,
                                None if local else cfg.rope_llama3_scaling)
            self._rope_cache[key] = tab
        return tab

    # ------------------------------------------------------------------ forward
    def forward(self, input_tokens, positions=None, cache=None, attention_mask=None, segment_ids=None,
                skip_lm_head: bool = False, output_hidden_states: bool = False, routed_experts=None):
        """`routed_experts` int [B, T, num_layers, top_k] replays the sampler's expert choice in every MoE layer
        (router replay, tunix/models/qwen3/model.py:895-939); entries < 0 leave a token to the layer's own router."""
        cfg = self.config
        B, T = input_tokens.shape
        emb_tokens = input_tokens
        if self.tp is not None and self.tp.world > 1:
            # sequence-parallel residual stream: this rank embeds its B/tp sequences; attention sees all of them
            if B % self.tp.world or cache is not None:
                raise ValueError("tensor parallelism needs the batch divisible by tp and no KV cache")
            n = B // self.tp.world
            emb_tokens = input_tokens[self.tp.rank * n:(self.tp.rank + 1) * n]
        cp = getattr(self, "cp", None)
        if cp is not None and cp.world > 1:
            # context parallel: every rank of the group got the same batch and keeps its slice of the sequence axis
            if positions is None:
                positions = torch.arange(T, device=input_tokens.device, dtype=torch.int32)[None].expand(B, T)
            emb_tokens, positions, segment_ids = cp.slice_seq(input_tokens), cp.slice_seq(positions), cp.slice_seq(segment_ids)
            routed_experts = cp.slice_seq(routed_experts)
            T = cp.local_len(T)
        x = F.embedding(emb_tokens, self.embed_tokens, math.sqrt(cfg.embed_dim) if cfg.embed_scale else 1.0)
        return self.forward_embeddings(x, positions=positions, cache=cache, attention_mask=attention_mask,
                                       segment_ids=segment_ids, skip_lm_head=skip_lm_head,
                                       output_hidden_states=output_hidden_states, batch_shape=(B, T),
                                       routed_experts=routed_experts)

    def forward_embeddings(self, x, positions=None, cache=None, attention_mask=None, segment_ids=None,
                           skip_lm_head: bool = False, output_hidden_states: bool = False, batch_shape=None,
                           routed_experts=None):
        """The decoder stack on input embeddings `x` (what `forward` runs after the token lookup; multimodal front
        ends call it with image soft tokens spliced in). `batch_shape` = (B, T) of the full batch when `x` is this
        rank's shard of it."""
        cfg = self.config
        B, T = batch_shape if batch_shape is not None else x.shape[:2]
        dev = x.device
        if positions is None:
            start = 0 if cache is None else cache[0]["end"]
            positions = torch.arange(start, start + T, device=dev, dtype=torch.int32)[None].expand(B, T)
        positions = positions.to(torch.int32).contiguous()
        new_cache = [] if cache is not None else None
        use_remat = cfg.remat_config != RematConfig.NONE and torch.is_grad_enabled() and cache is None
        hook = self.layer_grad_hook if (torch.is_grad_enabled() and cache is None) else None
        for i, layer in enumerate(self.layers):
            rope = self._rope(cfg.layer_type(i) == "local", dev)
            if hook is not None and x.requires_grad:
                x = _GradBoundary.apply(x, i, hook)
            forced = routed_experts[:, :, i] if (routed_experts is not None and cfg.is_moe) else None
            if use_remat and cfg.is_moe and not cfg.post_norms and getattr(layer.mlp, "ep", None) is not None \
                    and getattr(layer.mlp.ep, "fused", False):
                x = _moe_layer_split_remat(layer, x, positions, rope, segment_ids, attention_mask, forced)
            elif use_remat:
                x, _ = _torch_checkpoint(layer, x, positions, rope, None, segment_ids, attention_mask, forced,
                                         use_reentrant=False)
            else:
                x, c = layer(x, positions, rope, None if cache is None else cache[i], segment_ids, attention_mask, forced)
                if new_cache is not None:
                    new_cache.append(c)
        if hook is not None and x.requires_grad:
            x = _GradBoundary.apply(x, len(self.layers), hook)
        x = self.norm(x)
        if skip_lm_head or output_hidden_states:
            return x, new_cache
        return self.compute_final_logits(x), new_cache

    def compute_final_logits(self, hidden):
        return F.lm_head_logits(hidden, self.head_weight(), softcap=self.config.final_logit_softcap)

    def token_logprobs(self, hidden, targets, *, temperature: float = 1.0, want_entropy: bool = False,
                       chunk: Optional[int] = None):
        """log p(targets) from final hidden states without materialising [tokens, vocab] logits."""
        return F.lm_head_logprobs(hidden, self.head_weight(), targets, softcap=self.config.final_logit_softcap,
                                  temperature=temperature, want_entropy=want_entropy,
                                  chunk=chunk or self.config.logprob_chunk)

    def routed_experts_of_last_forward(self):
        """[B, T, num_layers, top_k] expert ids the MoE layers chose in the last forward (None for dense models)."""
        rows = [l.mlp.last_routed_experts for l in self.layers
                if isinstance(l.mlp, MoELayer) and l.mlp.last_routed_experts is not None]
        return torch.stack(rows, 2) if rows and len(rows) == len(self.layers) else None

    def aux_loss(self):
        """Sum of MoE router auxiliary losses of the last forward (None for dense models)."""
        losses = [l.mlp.last_aux_loss for l in self.layers
                  if isinstance(l.mlp, MoELayer) and l.mlp.last_aux_loss is not None]
        return sum(losses) if losses else None

    # -------------------------------------------------------------------- cache
    def init_cache(self, batch_size: int, cache_size: int, dtype=None, device=None):
        cfg = self.config
        dtype = dtype or cfg.dtype
        device = device or self.embed_tokens.device
        mk = lambda: torch.zeros(batch_size, cache_size, cfg.num_kv_heads, cfg.head_dim, dtype=dtype, device=device)  # noqa: E731
        return [{"k": mk(), "v": mk(), "seg": torch.zeros(batch_size, cache_size, dtype=torch.int32, device=device),
                 "end": 0} for _ in range(cfg.num_layers)]

    def get_model_input(self):
        dev = self.embed_tokens.device
        return {"input_tokens": torch.ones(2, 1, dtype=torch.int32, device=dev),
                "positions": torch.ones(2, 1, dtype=torch.int32, device=dev), "cache": None,
                "attention_mask": None}

    @property
    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())


def create_model(cfg: ModelConfig, device=None, seed: int = 0, init: bool = True) -> Transformer:
    """Random-init model of the given architecture (dummy-model creator of the reference:
    tunix/models/dummy_model_creator.py:29-92)."""
    if cfg.family == "gemma4":
        from .gemma4 import Gemma4Transformer
        model = Gemma4Transformer(cfg, device=device)
    else:
        model = Transformer(cfg, device=device)
    if init:
        model.init_weights(seed)
    return model
