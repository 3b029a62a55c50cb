"""PagedEngine: the in-framework GPU rollout engine (paged KV cache, CUDA-graphed decode).

It takes the place of the reference's vLLM / SGLang-JAX integrations (tunix/generate/vllm_sampler.py,
sglang_jax_sampler.py) and follows the page-table conventions of its host-side paged-KV prototype
(tunix/experimental/generate/single_type_kv_cache_manager.py, tiered_page_pool.py): fixed-size pages, a
free list, one page table row per running sequence.

Requests are batched continuously over `max_running_requests` slots (`_run`): a finished sequence frees its
slot and pages at the next check point and the next waiting request is prefilled into it.
  prefill  one pass over the left-padded prompts of the admitted requests with the tcgen05 flash-attention
           kernel; K / V of every layer are scattered into the pages by `kv_write` (padding is skipped);
  decode   every step is the same fixed sequence of kernel launches (embedding -> per layer RMSNorm, tcgen05
           GEMMs with narrow tiles, RoPE at device-resident positions, `kv_write`, `paged_decode` attention,
           GLU -> final norm -> lm_head GEMM in fp32 -> fused sampling kernel), all reading sequence lengths,
           the step counter and the page table from device memory, so the whole step is captured once in a
           CUDA graph and replayed; the host looks at the slots' done flags only every `check_every` steps.
Outputs match `Sampler` (`SamplerOutput` with ragged tokens, optional per-token log-probs).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np
import torch

from ..common.configs import CacheConfig
from ..ops import functional as F
from ..ops import kernels as K
from ..ops import sampling_kernels as S
from .base_sampler import BaseSampler, SamplerOutput
from .sampler import next_power_of_2, pad_prompts_left


class PagePool:
    """Device page pools for every layer plus the host-side bookkeeping.

    Which request holds which pages is kept by `experimental.generate.kv_cache_manager.KVCacheManager`: pages are
    reference counted, full pages are hashed by their token content (chained over the prefix), a released hashed
    page stays resident until the pool needs it (least recently released first), and a new request re-points to every
    cached page of its prompt's prefix (tunix/experimental/generate/single_type_kv_cache_manager.py:49-177). The
    table row of a slot is what the kernels read."""

    def __init__(self, cfg, num_pages: int, page_size: int, max_seqs: int, max_pages_per_seq: int, device, dtype,
                 prefix_caching: bool = True, kv_heads: Optional[int] = None):
        from ..experimental.generate import kv_cache_manager as kvm
        self.page_size, self.num_pages, self.max_pages = page_size, num_pages, max_pages_per_seq
        row = (kv_heads or cfg.num_kv_heads) * cfg.head_dim       # a tensor-parallel rank keeps its own kv heads only
        # zero-initialised: rows of a page that were never written must hold finite values
        self.k = [torch.zeros(num_pages, page_size, row, dtype=dtype, device=device) for _ in range(cfg.num_layers)]
        self.v = [torch.zeros(num_pages, page_size, row, dtype=dtype, device=device) for _ in range(cfg.num_layers)]
        self.table_host = np.full((max_seqs, max_pages_per_seq), -1, np.int32)
        self.table = torch.full((max_seqs, max_pages_per_seq), -1, dtype=torch.int32, device=device)
        self.Error = kvm.PagePoolError
        self.mgr = kvm.KVCacheManager(kvm.PagePool(num_pages), page_size, enable_prefix_caching=prefix_caching)
        self._rid: dict = {}            # slot -> request id inside the manager
        self._seq = 0
        self.hit_tokens = 0             # prompt tokens served from cached pages since construction
        self.prompt_tokens = 0

    @property
    def free_pages(self) -> int:
        return self.mgr.pool.num_free + len(self.mgr._lru)      # evictable cached pages count as free

    def _row(self, slot: int) -> None:
        self.table_host[slot] = self.mgr.page_table(self._rid[slot], self.max_pages)

    def open(self, slot: int, token_ids, n_new: int) -> int:
        """Pages for a new request in `slot`: its prompt plus `n_new` tokens. Returns how many leading prompt tokens
        already sit in cached pages. Raises `self.Error` when the pool cannot serve it (nothing is taken then)."""
        n = len(token_ids) + n_new
        if (n + self.page_size - 1) // self.page_size > self.max_pages:
            raise ValueError(f"sequence of {n} tokens does not fit the page table ({self.max_pages} pages)")
        self._seq += 1
        rid = f"{slot}#{self._seq}"
        _, cached = self.mgr.allocate_for_request(rid, token_ids, n_new)
        self._rid[slot] = rid
        self.mgr.cache_full_pages(rid, token_ids, len(token_ids))   # later requests may share these pages
        self._row(slot)
        self.hit_tokens += cached
        self.prompt_tokens += len(token_ids)
        return cached

    def grow(self, slot: int, total_tokens: int) -> None:
        """Make sure `slot` owns pages for `total_tokens` tokens. Raises `self.Error` when the pool is exhausted."""
        total_tokens = min(total_tokens, self.max_pages * self.page_size)
        before = len(self.mgr._req[self._rid[slot]])
        self.mgr.append_pages(self._rid[slot], total_tokens)
        if len(self.mgr._req[self._rid[slot]]) != before:
            self._row(slot)

    def publish(self, slot: int, token_ids) -> None:
        """Hash the pages that `token_ids` (prompt + generated) filled, so that a later turn of the same conversation
        finds them."""
        if slot in self._rid:
            self.mgr.cache_full_pages(self._rid[slot], token_ids, len(token_ids))

    def pages_of(self, slot: int) -> list:
        return [p.page_id for p in self.mgr._req[self._rid[slot]] if p is not None]

    def release(self, slot: int) -> None:
        rid = self._rid.pop(slot, None)
        if rid is None:
            return
        self.mgr.free_request(rid)
        self.table_host[slot, :] = -1

    def sync_table(self) -> None:
        self.table.copy_(torch.from_numpy(self.table_host), non_blocking=False)


class PagedEngine(BaseSampler):
    def __init__(self, transformer, tokenizer, cache_config: CacheConfig, page_size: int = 64,
                 max_running_requests: int = 64, use_cuda_graph: bool = True, check_every: int = 16,
                 use_pdl: bool = False, pack_weights: bool = True, num_pages: Optional[int] = None,
                 prefix_caching: bool = True, prefill_chunk: int = 0):
        self._model = transformer
        self.tokenizer = tokenizer
        self.cfg = transformer.config
        self.cache_size = cache_config.cache_size
        self.device = next(transformer.parameters()).device
        self.dtype = next(transformer.parameters()).dtype
        if self.device.type != "cuda" or self.dtype != torch.bfloat16:
            raise ValueError("PagedEngine runs bf16 models on CUDA; use Sampler elsewhere")
        if self.cfg.is_moe and getattr(transformer.layers[0].mlp, "ep", None) is not None:
            raise NotImplementedError("expert-parallel MoE decode goes through Sampler")
        if self.cfg.family == "gemma4":
            raise NotImplementedError("Gemma-4 decode (per-layer inputs, shared KV, 512-wide heads) goes through Sampler")
        # Tensor-parallel decode: a model sliced by `parallel.tp.apply_tensor_parallel` runs with this rank's heads and
        # MLP columns; the partial outputs of the o and down projections are summed over the group (one library
        # all-reduce of [sequences, D] each, captured in the decode graph). Embedding, norms and lm_head are whole on
        # every rank, so all ranks of the group compute the same logits and, with the same seed, sample the same
        # tokens: every rank of the group must be given the same requests in the same order.
        self.tp = getattr(transformer, "tp", None)
        self.tpw = self.tp.world if self.tp is not None else 1
        self.n_heads, self.n_kv = self.cfg.num_heads // self.tpw, self.cfg.num_kv_heads // self.tpw
        self.page_size = page_size
        self.max_running = max_running_requests
        self.use_graph = use_cuda_graph
        self.use_pdl = use_pdl      # programmatic dependent launch between the kernels of a decode step
        # the widest decode GEMMs (gate/up, lm_head) stream weights re-tiled into contiguous blocks
        # (ops.kernels.PackedWeight): a second copy of those weights, refreshed from the live parameters at the
        # start of every call. Measured at 64 rows on B200: 24576 x 4096 55 -> 51 us, 151936 x 4096 223 -> 205 us;
        # below ~16k weight rows a GEMM is bound by its fixed costs and the packed form does not pay.
        self.pack_weights = pack_weights
        self.pack_min_rows = 16384
        self._packed_on = False     # per call: the packed form wins up to 128 running sequences (one row of tiles)
        self._packed = None
        self.check_every = check_every
        self.max_pages_per_seq = (self.cache_size + page_size - 1) // page_size
        # pages in the pool: by default enough for every slot at full length (nothing ever queues for memory); a
        # smaller pool makes requests wait for pages and, when running sequences outgrow it, sends the youngest one
        # back to the queue
        self.num_pages = num_pages
        self.prefix_caching = prefix_caching
        self.prefill_chunk = prefill_chunk      # > 0: prompts are prefilled in pieces of at most this many tokens
        self.preemptions = 0
        self.forbidden: Optional[torch.Tensor] = None
        self.pool: Optional[PagePool] = None
        self._graph = None
        self._graph_key = None

    # ----------------------------------------------------------------- plumbing
    @property
    def transformer(self):
        return self._model

    def tokenize(self, input_string: str):
        ids = self.tokenizer.encode(input_string)
        bos = self.tokenizer.bos_id()
        if bos is not None and (not ids or ids[0] != bos):
            ids = [bos] + list(ids)
        return np.asarray(ids, np.int64)

    @torch.no_grad()
    def update_params(self, updated_weights: dict, filter_types=None) -> None:
        own = dict(self._model.named_parameters())
        for name, w in updated_weights.items():
            if own[name].data_ptr() != w.data_ptr():
                own[name].copy_(w.to(own[name].device, own[name].dtype))

    def delete_cache(self) -> None:
        self.pool = None
        self._graph = None

    def reinitialize_cache(self) -> None:
        self._ensure_pool(self.max_running)

    def _ensure_pool(self, n_seqs: int) -> None:
        if self.pool is None:
            pages = self.num_pages or self.max_running * self.max_pages_per_seq
            self.pool = PagePool(self.cfg, pages, self.page_size, self.max_running, self.max_pages_per_seq, self.device,
                                 self.dtype, self.prefix_caching, kv_heads=self.n_kv)

    # ---------------------------------------------------------------- the model
    @staticmethod
    def _fused_weight(mods):
        """One [sum(out_i), in] view over the weights of `mods`, so that projections sharing an input run as a
        single GEMM. Weights already back to back in one storage (the optimizer's flat buffer lays q/k/v and
        gate/up out that way) are viewed in place; weights that own their storage are moved, once, into a joint
        tensor and stay views of it. Anything else (bias, LoRA, quantised base, foreign layout) returns None and
        the caller runs the projections one by one."""
        if any(m.quant is not None or m.bias is not None or (m.lora_a is not None and m.lora_enabled) for m in mods):
            return None
        ws = [m.weight for m in mods]
        cols = ws[0].shape[1]
        if any(w.shape[1] != cols or not w.is_contiguous() for w in ws):
            return None
        rows = sum(w.shape[0] for w in ws)
        base = ws[0].data
        off, adjacent = base.storage_offset(), True
        for w in ws:
            if w.untyped_storage().data_ptr() != base.untyped_storage().data_ptr() or w.storage_offset() != off:
                adjacent = False
                break
            off += w.numel()
        if adjacent:
            return base.as_strided((rows, cols), (cols, 1), base.storage_offset())
        esz = base.element_size()
        if any(w.untyped_storage().nbytes() != w.numel() * esz for w in ws):
            return None     # views of someone else's buffer: leave them where they are
        joint = torch.empty((rows, cols), dtype=base.dtype, device=base.device)
        r = 0
        for w in ws:
            joint[r:r + w.shape[0]].copy_(w.data)
            w.data = joint[r:r + w.shape[0]]
            r += w.shape[0]
        return joint

    def _fuse_all(self):
        self._wqkv, self._wgu = [], []
        for layer in self._model.layers:
            at = layer.self_attn
            self._wqkv.append(self._fused_weight([at.q_proj, at.k_proj, at.v_proj]))
            # a mixture-of-experts block keeps its stacked expert weights and runs through the grouped GEMM
            self._wgu.append(None if self.cfg.is_moe else self._fused_weight([layer.mlp.gate_proj, layer.mlp.up_proj]))

    @staticmethod
    def _plain(mod) -> bool:
        return mod.quant is None and mod.bias is None and not (mod.lora_a is not None and mod.lora_enabled)

    def _pack_all(self) -> None:
        """(Re)pack the weights the decode step multiplies by. The buffers are allocated once, so a captured
        decode graph keeps pointing at them; a projection with bias, LoRA or a quantised base is left to the
        unpacked path (entry None)."""
        if not self.pack_weights:
            self._packed = None
            return
        srcs = []
        for i, layer in enumerate(self._model.layers):
            at, mlp = layer.self_attn, layer.mlp
            dense = not self.cfg.is_moe
            srcs.append({"qkv": self._wqkv[i], "o": at.o_proj.weight.data if self._plain(at.o_proj) else None,
                         "gu": self._wgu[i],
                         "down": mlp.down_proj.weight.data if dense and self._plain(mlp.down_proj) else None})
        srcs.append({"head": self._model.head_weight()})
        for src in srcs:
            for name, w in src.items():
                if w is not None and (w.shape[0] < self.pack_min_rows or w.dtype != torch.bfloat16 or w.shape[1] % 8):
                    src[name] = None
        fresh = self._packed is None or len(self._packed) != len(srcs)
        if not fresh:
            for have, src in zip(self._packed, srcs):
                for name, w in src.items():
                    pw = have.get(name)
                    if (pw is None) != (w is None) or (pw is not None and (pw.N, pw.K) != tuple(w.shape)):
                        fresh = True
        if fresh:
            # the fused gate / up weight is packed with its rows interleaved, so that the GEMM's epilogue applies the
            # gated activation (no [rows, 2F] intermediate, no separate activation kernel)
            self._packed = [{name: (K.PackedWeight(w, glu=(name == "gu" and w.shape[0] % 32 == 0)) if w is not None else None)
                             for name, w in src.items()} for src in srcs]
            self._graph = None          # a captured graph points at the old buffers
            return
        for have, src in zip(self._packed, srcs):
            for name, w in src.items():
                if have[name] is not None:
                    have[name].refresh(w)

    def _pk(self, i, name):
        return self._packed[i].get(name) if self._packed is not None and self._packed_on else None

    def _rope(self, i):
        return self._model._rope(self.cfg.layer_type(i) == "local", self.device)

    def _attn_in(self, layer, h2, positions_flat, i):
        """Projections + QK-norm + RoPE on flat rows h2 [n, D] -> q [n,N,H], k [n,K,H], v [n,K*H]."""
        cfg, at = self.cfg, layer.self_attn
        N, KH, H = self.n_heads, self.n_kv, cfg.head_dim
        q = F.linear(h2, at.q_proj.base_weight(), at.q_proj.bias).view(-1, N, H)
        k = F.linear(h2, at.k_proj.base_weight(), at.k_proj.bias).view(-1, KH, H)
        v = F.linear(h2, at.v_proj.base_weight(), at.v_proj.bias)
        for proj, name in ((at.q_proj, "q"), (at.k_proj, "k"), (at.v_proj, "v")):
            if proj.lora_a is not None and proj.lora_enabled:
                delta = F.linear(F.linear(h2, proj.lora_a), proj.lora_b) * proj.lora_scale
                if name == "q":
                    q = q + delta.view_as(q)
                elif name == "k":
                    k = k + delta.view_as(k)
                else:
                    v = v + delta
        if cfg.qk_norm:
            q = at.q_norm(q)
            k = at.k_norm(k)
        cos, sin = self._rope(i)
        K.rope_(q, positions_flat, cos, sin)
        K.rope_(k, positions_flat, cos, sin)
        return q, k, v

    def _lin(self, mod, x, residual=None):
        return mod(x, residual=residual)   # Linear.forward handles LoRA; no autograd under no_grad

    def _mlp(self, layer, i, h, residual=None, decode=False):
        wgu = self._wgu[i]
        if wgu is None and self.tpw > 1:
            raise NotImplementedError("tensor-parallel decode needs plain MLP weights (no adapters, no quantised base, no MoE)")
        if wgu is None:
            if self.cfg.is_moe and h.dim() == 2:      # decode rows: the expert block wants [batch, time, D]
                r3 = residual[:, None] if residual is not None else None
                return layer.mlp(h[:, None], residual=r3)[:, 0]
            return layer.mlp(h, residual=residual)
        Fd = wgu.shape[0] // 2
        h2 = h.reshape(-1, h.shape[-1])
        pgu = self._pk(i, "gu") if decode else None
        kind = K.GLU_SILU if layer.mlp.kind == "silu" else K.GLU_GELU
        if pgu is not None and pgu.glu:
            a = K.gemm_packed(h2, pgu, glu=kind)
        else:
            gu = K.gemm_packed(h2, pgu) if pgu is not None else F.linear(h2, wgu)
            a = K.glu_fwd(gu[:, :Fd], gu[:, Fd:], kind)
        pdown = self._pk(i, "down") if decode else None
        if self.tpw > 1:
            y = K.gemm_packed(a, pdown) if pdown is not None else layer.mlp.down_proj(a)
            return self._tp_sum(y, None if residual is None else residual.reshape(y.shape)).view(*h.shape[:-1], -1)
        if pdown is not None:
            r2 = residual.reshape(-1, residual.shape[-1]) if residual is not None else None
            return K.gemm_packed(a, pdown, residual=r2).view(*h.shape[:-1], -1)
        return layer.mlp.down_proj(a.view(*h.shape[:-1], Fd), residual=residual)

    def _tp_sum(self, y, residual):
        """Sum the ranks' partial projection outputs (in place) and add the residual once."""
        import torch.distributed as dist
        dist.all_reduce(y, group=self.tp.group)
        return y if residual is None else y.add_(residual)

    def _mlp_and_norms(self, layer, i, x, attn_out, decode=False):
        cfg = self.cfg
        if cfg.post_norms:
            x = x + layer.post_attn_norm(attn_out)
            m = self._mlp(layer, i, layer.post_attention_layernorm(x), decode=decode)
            return x + layer.post_ffw_norm(m)
        x = attn_out          # o_proj already added the residual
        return self._mlp(layer, i, layer.post_attention_layernorm(x), residual=x, decode=decode)

    def _prefill(self, toks, positions, seg, slots, prev_len=None, write_from=None):
        """toks [B,P] left padded: the prompt tokens this call computes. `prev_len` [B] (or None): tokens of each row
        that already sit in its pages (a prefix-cache hit, or the earlier chunks of a long prompt): their K/V are
        gathered from the pages and attended to. K/V of this call's tokens are written at positions >= write_from
        (a row never rewrites pages it shares). Returns the hidden state of the last position [B, D]."""
        cfg, pool = self.cfg, self.pool
        B, P = toks.shape
        KH, H = self.n_kv, cfg.head_dim
        x = F.embedding(toks, self._model.embed_tokens, math.sqrt(cfg.embed_dim) if cfg.embed_scale else 1.0)
        pos_flat = positions.reshape(-1).contiguous()
        valid = seg.reshape(-1) > 0
        if write_from is not None:
            valid = valid & (pos_flat >= write_from.repeat_interleave(P))
        wpos = torch.where(valid, pos_flat, torch.full_like(pos_flat, -1))
        seq_ids = slots.repeat_interleave(P)
        Tc, pidx, seg_k = 0, None, seg
        if prev_len is not None:
            Tc = (int(prev_len.max()) + pool.page_size - 1) // pool.page_size * pool.page_size
        if Tc > 0:
            pidx = pool.table[slots.long(), :Tc // pool.page_size].clamp(min=0).long()          # [B, pages]
            seg_c = (torch.arange(Tc, device=toks.device)[None] < prev_len[:, None]).to(torch.int32)
            seg_k = torch.cat([seg_c, seg], 1).contiguous()
        for i, layer in enumerate(self._model.layers):
            h = layer.input_layernorm(x)
            q, k, v = self._attn_in(layer, h.view(B * P, -1), pos_flat, i)
            K.kv_write(k.view(B * P, -1), v, seq_ids, wpos, pool.table, pool.page_size, pool.k[i], pool.v[i])
            at = layer.self_attn
            k4, v4 = k.view(B, P, KH, H), v.view(B, P, KH, H)
            if Tc > 0:
                k4 = torch.cat([pool.k[i][pidx].view(B, Tc, KH, H), k4], 1)
                v4 = torch.cat([pool.v[i][pidx].view(B, Tc, KH, H), v4], 1)
            o = F.attention(q.view(B, P, self.n_heads, H), k4, v4, scale=at.scale, causal=True, window=at.window,
                            softcap=cfg.attn_logit_softcap, q_off=Tc if Tc > 0 else None, seg_q=seg, seg_k=seg_k)
            o = o.reshape(B, P, -1)
            if self.tpw > 1:
                a = self._tp_sum(at.o_proj(o), None if cfg.post_norms else x)
            else:
                a = at.o_proj(o, residual=None if cfg.post_norms else x)
            x = self._mlp_and_norms(layer, i, x, a)
        return self._model.norm(x[:, -1])

    def _decode_step(self, st) -> None:
        """One token for every sequence of the wave. `st` holds the static device buffers."""
        cfg, pool = self.cfg, self.pool
        B = st["tokens"].shape[0]
        N, KH, H = self.n_heads, self.n_kv, cfg.head_dim
        x = F.embedding(st["tokens"], self._model.embed_tokens, math.sqrt(cfg.embed_dim) if cfg.embed_scale else 1.0)
        pos = st["positions"]           # position of the token being fed = seq_len before it is appended
        lens = st["seq_lens"]           # length including that token
        for i, layer in enumerate(self._model.layers):
            h = layer.input_layernorm(x)
            at = layer.self_attn
            if self._wqkv[i] is not None:
                pq = self._pk(i, "qkv")
                qkv = K.gemm_packed(h, pq) if pq is not None else F.linear(h, self._wqkv[i])
                cos, sin = self._rope(i)
                qn, kn = (at.q_norm, at.k_norm) if cfg.qk_norm else (None, None)
                K.qkv_post(qkv, st["slots"], pos, qn.weight if qn is not None else None,
                           kn.weight if kn is not None else None, cfg.norm_eps, cfg.norm_add_one, cos, sin, pool.table,
                           pool.page_size, pool.k[i], pool.v[i], N, KH, H)
                q = qkv[:, :N * H].view(B, N, H)
            else:
                q, k, v = self._attn_in(layer, h, pos, i)
                K.kv_write(k.view(B, -1), v, st["slots"], pos, pool.table, pool.page_size, pool.k[i], pool.v[i])
            o = K.paged_decode(q, pool.k[i], pool.v[i], pool.table, st["slots"], lens, num_kv_heads=KH,
                               page_size=pool.page_size, max_ctx=self.cache_size, scale=at.scale,
                               softcap=cfg.attn_logit_softcap, window=at.window, workspace=st["ws"], split_tokens=st["split"])
            po = self._pk(i, "o")
            if self.tpw > 1:
                a = K.gemm_packed(o.view(B, N * H), po) if po is not None else at.o_proj(o.view(B, N * H))
                a = self._tp_sum(a, None if cfg.post_norms else x)
            elif po is not None:
                a = K.gemm_packed(o.view(B, N * H), po, residual=None if cfg.post_norms else x)
            else:
                a = at.o_proj(o.view(B, N * H), residual=None if cfg.post_norms else x)
            x = self._mlp_and_norms(layer, i, x, a, decode=True)
        hlast = self._model.norm(x)
        self._sample_into(hlast, st)

    def _logits(self, hlast, out=None):
        ph = self._pk(len(self._model.layers), "head")
        if ph is not None:
            logits = K.gemm_packed(hlast, ph, out=out, out_dtype=torch.float32)
        else:
            logits = K.gemm(hlast, self._model.head_weight(), out=out, out_dtype=torch.float32)
        return logits          # raw: the final soft-cap is applied by the sampling kernel (`_sample`)

    def _sample(self, logits, st, out_tokens, out_logprobs) -> None:
        p = st["params"]
        S.sample(logits, p["temperature"], p["top_p"], p["top_k"], p["seed"], 0, want_logprob=True,
                 out_tokens=out_tokens, out_logprobs=out_logprobs, step_tensor=st["step"],
                 softcap=float(self.cfg.final_logit_softcap or 0.0), forbidden=self.forbidden)

    def _sample_into(self, hlast, st) -> None:
        """Sample one token per slot of the running batch and advance the slots that are still generating. A
        finished (or empty) slot idles: position -1 and length 0 make the next step write no K/V and attend to
        nothing, and its output goes to the spare last column."""
        logits = self._logits(hlast, out=st["logits"])
        self._sample(logits, st, st["next"], st["next_lp"])
        # append, mark finished slots, and set up the next step's token / position / length: one kernel for all slots
        K.decode_advance(st, st["pad_id"])

    # --------------------------------------------------------------------- call
    @torch.no_grad()
    def __call__(self, input_strings=None, max_generation_steps: int = 0, max_prompt_length: Optional[int] = None,
                 echo: bool = False, return_logits: bool = False, return_logprobs: bool = False,
                 eos_tokens: Optional[Sequence[int]] = None, forbidden_tokens=None, temperature: float = 0.0,
                 top_p: Optional[float] = None, top_k: Optional[int] = None, beam_size=None, seed: Optional[int] = None,
                 pad_output: bool = False, *, prompt_token_ids=None) -> SamplerOutput:
        if beam_size or return_logits or echo:
            raise NotImplementedError("beam search, logits and echo are served by Sampler")
        self.forbidden = torch.as_tensor(sorted({int(t) for t in forbidden_tokens}), dtype=torch.int32, device=self.device) \
            if forbidden_tokens else None
        if (input_strings is None) == (prompt_token_ids is None):
            raise ValueError("give exactly one of input_strings / prompt_token_ids")
        if isinstance(input_strings, str):
            input_strings = [input_strings]
        rows = [list(r) for r in prompt_token_ids] if prompt_token_ids is not None else \
            [self.tokenize(s).tolist() for s in input_strings]
        eos_ids = list(eos_tokens) if eos_tokens else [self.tokenizer.eos_id()]
        pad_id = self.tokenizer.pad_id()
        plen = max_prompt_length if max_prompt_length else next_power_of_2(max(len(r) for r in rows))
        if plen + max_generation_steps > self.cache_size:
            raise ValueError("prompt + generation exceeds the configured cache size")
        was_training = self._model.training
        self._model.eval()
        prompts_all, plens_all = pad_prompts_left(rows, plen, pad_id)
        self._fuse_all()
        self._packed_on = self.pack_weights and min(self.max_running, len(rows)) <= 128
        if self._packed_on:
            self._pack_all()
        from .. import _lib
        _lib.register_cuda_sigs({"tb_set_pdl": [_lib.I]})
        _lib.cuda().tb_set_pdl(1 if self.use_pdl else 0)
        try:
            gen, lps = self._run(prompts_all, plens_all, max_generation_steps, eos_ids, pad_id, temperature, top_p, top_k,
                                 seed or 0)
        finally:
            _lib.cuda().tb_set_pdl(0)
            self._model.train(was_training)
        tokens, texts, lp_out = [], [], []
        for b in range(gen.shape[0]):
            row = gen[b]
            stop = len(row)
            for i, t in enumerate(row):
                if t in eos_ids:
                    stop = i + 1
                    break
            row = row[:stop]
            if pad_output:
                row = np.concatenate([row, np.full(max_generation_steps - len(row), pad_id, row.dtype)])
            tokens.append(row)
            texts.append(self.tokenizer.decode([t for t in row[:stop] if t not in eos_ids and t != pad_id]))
            lp_out.append(lps[b, :stop].tolist())
        return SamplerOutput(text=texts, logits=None, tokens=np.stack(tokens) if pad_output else tokens,
                             padded_prompt_tokens=prompts_all, logprobs=lp_out if return_logprobs else None,
                             prompt_lengths=np.asarray(plens_all))

    def _new_state(self, B, max_steps, eos_ids, pad_id, temperature, top_p, top_k, seed):
        dev = self.device
        split = K.decode_split_tokens(B, self.n_kv, self.cache_size)
        splits = (self.cache_size + split - 1) // split
        N, H, V = self.n_heads, self.cfg.head_dim, self.cfg.vocab_size
        i64 = dict(dtype=torch.int64, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        return {
            "tokens": torch.zeros(B, **i64),
            "positions": torch.full((B,), -1, **i32),             # -1 / 0: an empty slot
            "seq_lens": torch.zeros(B, **i32),
            "slots": torch.arange(B, **i32), "done": torch.ones(B, dtype=torch.bool, device=dev),
            "next": torch.zeros(B, **i64), "next_lp": torch.zeros(B, device=dev),
            "out_tokens": torch.full((B, max_steps + 1), pad_id, **i64),      # last column: writes of idle slots
            "out_lp": torch.zeros((B, max_steps + 1), device=dev),
            "out_pos": torch.zeros(B, **i64),
            "limit": torch.full((B,), max_steps, **i64),          # tokens the slot's request may generate
            "dump_col": torch.full((B,), max_steps, **i64),
            "neg1": torch.full((B,), -1, **i32), "zero": torch.zeros(B, **i32),
            "logits": torch.empty(B, V, dtype=torch.float32, device=dev),
            "step": torch.zeros(1, **i32),
            "pad": torch.full((B,), pad_id, **i64), "pad_id": int(pad_id),
            "eos": torch.as_tensor(eos_ids, **i64),
            "ws": (torch.empty(B * N * splits * H, dtype=torch.float32, device=dev),
                   torch.empty(B * N * splits * 2, dtype=torch.float32, device=dev)),
            "params": {"temperature": temperature, "top_p": top_p, "top_k": top_k, "seed": seed},
            "split": split,
        }

    def _run(self, toks_np, lens_np, max_steps, eos_ids, pad_id, temperature, top_p, top_k, seed):
        """All requests of one call through the continuous-batching loop. toks_np [n, P] left-padded prompts,
        lens_np [n]. Returns (tokens [n, max_steps], logprobs [n, max_steps])."""
        n_req = toks_np.shape[0]
        out_tok = np.full((n_req, max_steps), pad_id, np.int64)
        out_lp = np.zeros((n_req, max_steps), np.float32)
        if max_steps == 0 or n_req == 0:
            return out_tok, out_lp
        B = min(self.max_running, n_req)
        st = self._new_state(B, max_steps, eos_ids, pad_id, temperature, top_p, top_k, seed)
        waiting = list(range(n_req))[::-1]          # pop() takes the next request in order

        class Source:
            def take(self, n_free):
                reqs = [waiting.pop() for _ in range(min(n_free, len(waiting)))]
                return [(r, toks_np[r], int(lens_np[r]), max_steps) for r in reqs]

            def give_back(self, items):
                waiting.extend(r for r, *_ in reversed(items))      # back to the head of the queue, order kept

            def more_waiting(self):
                return bool(waiting)

            def deliver(self, r, toks, lps):
                out_tok[r, :len(toks)] = toks
                out_lp[r, :len(lps)] = lps

            def idle(self):
                return False                        # nothing running and nothing waiting: the call is over

        self._loop(st, B, max_steps, pad_id, Source())
        return out_tok, out_lp

    def _loop(self, st, B, max_steps, pad_id, source) -> None:
        """Continuous batching over B slots. A slot whose sequence has finished (end-of-sequence token or its
        token limit) is harvested at the next check point (every `check_every` decode steps at most), its pages go
        back to the pool, and the next waiting request is prefilled into it while the other slots keep their
        state. The decode step always runs over all slots (one captured graph); idle slots cost a row of the
        GEMMs and no attention work.

        Pages are handed out as sequences grow: a request is admitted with pages for its prompt and the steps up to
        the next check point, and every check point tops the running slots up. A request that finds no room stays in
        the queue; when running sequences outgrow the pool, the one with the least progress goes back to the head of
        the queue (its pages are released, it is generated again from its prompt later) instead of failing the call.
        Prompt pages are shared through the prefix cache: a request whose prompt starts with tokens that already sit
        in cached pages (the other generations of its GRPO group, an earlier turn of its conversation) prefills only
        what is left.

        `source` hands out requests and takes results: take(n_free) -> [(id, padded prompt row, prompt length,
        token limit)], give_back(items), more_waiting(), deliver(id, tokens, logprobs), and idle(), called when no
        slot is busy and take() returned nothing: it may block for new work and returns False to end the loop."""
        dev = self.device
        self._ensure_pool(B)
        pool = self.pool
        for s in range(self.max_running):
            pool.release(s)
        i64 = dict(dtype=torch.int64, device=dev)
        slot_req = [None] * B
        slot_item = [None] * B                      # the request as take() gave it (for give_back)
        slot_cnt = [0] * B                          # tokens a slot's request has produced at most (host-side bound)
        slot_lim = [0] * B
        slot_plen = [0] * B
        graph = None

        def prompt_ids(item):
            _rid, row, ln, _lim = item
            return [int(t) for t in row[len(row) - ln:]]

        def idle_slot(s):
            st["done"][s] = True
            st["positions"][s] = -1
            st["seq_lens"][s] = 0

        while True:
            # ---- check point: harvest finished slots, admit waiting requests (repeats while an admitted request
            # finishes with its very first token)
            while True:
                done_h = st["done"].cpu().numpy()
                fin = [s for s in range(B) if slot_req[s] is not None and done_h[s]]
                if fin:
                    ix = torch.as_tensor(fin, **i64)
                    toks_h = st["out_tokens"][ix, :max_steps].cpu().numpy()
                    lps_h = st["out_lp"][ix, :max_steps].cpu().numpy()
                    cnt_h = st["out_pos"][ix].cpu().numpy()
                    for j, s in enumerate(fin):
                        c = int(cnt_h[j])
                        source.deliver(slot_req[s], toks_h[j, :c], lps_h[j, :c])
                        # the K/V of everything but the last sampled token is in the pages: a follow-up turn finds it
                        pool.publish(s, prompt_ids(slot_item[s]) + [int(t) for t in toks_h[j, :max(c - 1, 0)]])
                        slot_req[s] = slot_item[s] = None
                        pool.release(s)
                if getattr(source, "streaming", False):          # someone listens: report what the running requests have so far
                    run = [s for s in range(B) if slot_req[s] is not None and not done_h[s]]
                    if run:
                        rx = torch.as_tensor(run, **i64)
                        p_cnt = st["out_pos"][rx].cpu().numpy()
                        p_tok = st["out_tokens"][rx, :max_steps].cpu().numpy()
                        p_lp = st["out_lp"][rx, :max_steps].cpu().numpy()
                        for j, s in enumerate(run):
                            c = int(p_cnt[j])
                            if c > 0:
                                source.progress(slot_req[s], p_tok[j, :c], p_lp[j, :c])
                free = [s for s in range(B) if slot_req[s] is None]
                new = source.take(len(free)) if free else []
                if not new:
                    break
                admitted = []                        # (slot, item, cached tokens)
                for n_i, item in enumerate(new):
                    s = free[len(admitted)]
                    lim = max(1, min(int(item[3]), max_steps))
                    try:
                        cached = pool.open(s, prompt_ids(item), min(lim, self.check_every) + 1)
                    except pool.Error:
                        source.give_back(new[n_i:])   # no room now: they wait for pages
                        break
                    slot_req[s], slot_item[s] = item[0], item
                    slot_cnt[s], slot_lim[s], slot_plen[s] = 1, lim, item[2]
                    admitted.append((s, item, cached))
                if not admitted:
                    if all(r is None for r in slot_req):
                        raise RuntimeError(f"the page pool ({pool.num_pages} pages of {pool.page_size} tokens) cannot hold "
                                           f"a single request of {new[0][2]} prompt tokens")
                    break
                pool.sync_table()
                # requests whose cached pages are written by another request of this admission pass wait for that prefill
                produced: dict = {}
                waves: dict = {}
                for s, item, cached in admitted:
                    pages = pool.pages_of(s)
                    n_cached = cached // pool.page_size
                    wave = 1 + max((produced.get(pg, -1) for pg in pages[:n_cached]), default=-1)
                    for pg in pages[n_cached:item[2] // pool.page_size]:
                        produced.setdefault(pg, wave)
                    waves.setdefault(wave, []).append((s, item, cached))
                for wave in sorted(waves):
                    grp = waves[wave]
                    self._admit(st, [s for s, _, _ in grp], np.stack([it[1] for _, it, _ in grp]),
                                np.asarray([it[2] for _, it, _ in grp]), pad_id, [slot_lim[s] for s, _, _ in grp],
                                [c for _, _, c in grp])
            if all(r is None for r in slot_req):
                if source.idle():
                    continue
                break
            # ---- decode until the next check point; no slot can run past its token limit, which bounds the steps
            # to the next look at the done flags
            if graph is None and self.use_graph and max_steps > 2:
                graph = self._capture(st)
            running = [s for s in range(B) if slot_req[s] is not None]
            left = [slot_lim[s] - slot_cnt[s] for s in running]
            n_steps = max(1, min(self.check_every, min(left) if source.more_waiting() else max(left)))
            # pages for the steps ahead; when the pool runs dry the youngest sequence makes room
            changed = False
            while True:
                try:
                    for s in running:
                        before = len(pool.pages_of(s))
                        pool.grow(s, slot_plen[s] + min(slot_cnt[s] + n_steps, slot_lim[s]) + 1)
                        changed |= len(pool.pages_of(s)) != before
                    break
                except pool.Error:
                    if len(running) <= 1:
                        raise RuntimeError("the page pool cannot hold one sequence at its full length") from None
                    victim = min(running, key=lambda s: (slot_cnt[s], -s))
                    source.give_back([slot_item[victim]])
                    idle_slot(victim)
                    pool.release(victim)
                    slot_req[victim] = slot_item[victim] = None
                    running.remove(victim)
                    self.preemptions += 1
                    changed = True
            if changed:
                pool.sync_table()
            for _ in range(n_steps):
                if graph is not None:
                    graph.replay()
                else:
                    self._decode_step(st)
            for s in range(B):
                slot_cnt[s] += n_steps

    def _admit(self, st, slots_list, toks_np, lens_np, pad_id, limits, cached=None) -> None:
        """Prefill the given prompts into their slots, sample each one's first token and set the slot state.
        `cached[i]` leading tokens of prompt i already sit in (shared) pages and are not computed again, except that
        the last prompt token always is: its hidden state gives the first sampled token. Long remainders are
        prefilled in pieces of `prefill_chunk` tokens, each attending to the pages written before it."""
        dev = self.device
        g = len(slots_list)
        ps = self.pool.page_size
        cached = [0] * g if cached is None else list(cached)
        lens_l = [int(x) for x in lens_np]
        use = [min(c, (ln - 1) // ps * ps) for c, ln in zip(cached, lens_l)]       # tokens taken from the pages
        newlen = [ln - u for ln, u in zip(lens_l, use)]
        Pn = max(newlen)
        P = toks_np.shape[1]
        new_np = np.full((g, Pn), pad_id, np.int64)
        for i in range(g):
            new_np[i, Pn - newlen[i]:] = toks_np[i, P - newlen[i]:]
        toks = torch.from_numpy(new_np).to(dev)
        nl = torch.as_tensor(newlen, device=dev)
        prev = torch.as_tensor(use, dtype=torch.int32, device=dev)
        wfrom = torch.as_tensor(cached, dtype=torch.int32, device=dev)
        lens = torch.as_tensor(lens_l, device=dev)
        seg = (torch.arange(Pn, device=dev)[None] >= (Pn - nl)[:, None]).to(torch.int32)
        positions = (torch.clamp(torch.cumsum(seg, -1) - 1, min=0) + prev[:, None]).to(torch.int32)
        slots = torch.as_tensor(slots_list, dtype=torch.int32, device=dev)
        chunk = self.prefill_chunk if self.prefill_chunk and self.prefill_chunk > 0 else Pn
        hlast = None
        for c0 in range(0, Pn, chunk):
            c1 = min(Pn, c0 + chunk)
            before = prev + seg[:, :c0].sum(-1).to(torch.int32)                     # tokens of each row already in pages
            use_prev = before if (c0 > 0 or any(use)) else None
            hlast = self._prefill(toks[:, c0:c1].contiguous(), positions[:, c0:c1].contiguous(),
                                  seg[:, c0:c1].contiguous(), slots, use_prev, wfrom)
        logits = self._logits(hlast)
        nxt = torch.zeros(g, dtype=torch.int64, device=dev)
        nlp = torch.zeros(g, device=dev)
        self._sample(logits, st, nxt, nlp)
        ix = slots.to(torch.int64)
        lim = torch.as_tensor(limits, dtype=torch.int64, device=dev)
        st["out_tokens"][ix] = pad_id
        st["out_tokens"][ix, 0] = nxt
        st["out_lp"][ix, 0] = nlp
        st["out_pos"][ix] = 1
        st["limit"][ix] = lim
        done = (nxt[:, None] == st["eos"]).any(-1) | (lim <= 1)
        st["done"][ix] = done
        st["tokens"][ix] = nxt
        # token 0 came from the prefill's last hidden state; it is fed at position `len`
        st["positions"][ix] = torch.where(done, st["neg1"][ix], lens.to(torch.int32))
        st["seq_lens"][ix] = torch.where(done, st["zero"][ix], (lens + 1).to(torch.int32))

    def _capture(self, st):
        """Warm the decode path once outside capture (lazy kernel attribute setup, tensor-map cache), then capture
        one step; the state the warm-up and the capture touched is put back."""
        keys = ("tokens", "positions", "seq_lens", "done", "out_tokens", "out_lp", "out_pos", "step")
        snap = {k: st[k].clone() for k in keys}
        self._decode_step(st)
        for k, v in snap.items():
            st[k].copy_(v)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        # thread-local capture: other threads of the process (a trainer, another engine) keep using CUDA meanwhile
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            self._decode_step(st)
        for k, v in snap.items():
            st[k].copy_(v)
        return graph


class EngineServer:
    """Server mode of `PagedEngine`: any thread submits single requests, which join the running batch at the next
    check point instead of waiting for a batch to be assembled (the role of the reference's vLLM server mode,
    tunix/generate/vllm_sampler.py:281-355, that agentic rollouts depend on: one prompt per call,
    tunix/rl/agentic/agentic_rl_learner.py:441-500).

    One loop thread owns the engine. Sampling parameters, the prompt window and the token limit's upper bound are
    fixed per server (they shape the captured decode step); `max_tokens` is per request. `pause()` stops admission
    and returns once the running requests have been delivered, so that weights can be updated in place;
    `resume()` re-reads them (fused views, packed copies) and admits again."""

    def __init__(self, engine: PagedEngine, *, max_new_tokens: int, max_prompt_length: int, temperature: float = 0.0,
                 top_p: Optional[float] = None, top_k: Optional[int] = None, seed: int = 0,
                 eos_tokens: Optional[Sequence[int]] = None):
        import collections
        import threading
        if max_prompt_length + max_new_tokens > engine.cache_size:
            raise ValueError("prompt + generation exceeds the configured cache size")
        self.engine = engine
        self.max_new_tokens = int(max_new_tokens)
        self.P = int(max_prompt_length)
        self.pad_id = engine.tokenizer.pad_id()
        self._eos = list(eos_tokens) if eos_tokens else [engine.tokenizer.eos_id()]
        self._sampling = (temperature, top_p, top_k, seed)
        self._cv = threading.Condition()
        self._queue = collections.deque()
        self._futures: dict = {}
        self._callbacks: dict = {}              # request id -> [callback, tokens already reported]
        self._next_id = 0
        self._paused = False
        self._closed = False
        self._drained = threading.Event()
        self._error: Optional[BaseException] = None
        self.admitted = 0
        self._thread = threading.Thread(target=self._serve, name="tunix-b200-engine-server", daemon=True)
        self._thread.start()

    # ------------------------------------------------------------------ client side
    streams = True          # `submit(..., on_tokens=...)` reports tokens while a request is still running

    def submit(self, prompt_token_ids, max_tokens: Optional[int] = None, on_tokens=None):
        """Queue one request; the returned future resolves to (tokens int64 [n], logprobs float32 [n]).

        `on_tokens(new_tokens, new_logprobs)` is called from the engine's loop thread with the tokens produced since
        the previous call, at every check point of the decode loop and once more when the request finishes (so the
        pieces concatenate to the final result). It must return quickly. A request that the engine pre-empts for lack
        of pages starts again from its prompt; pieces already reported are not reported again."""
        from concurrent.futures import Future
        ids = list(prompt_token_ids)[-self.P:]
        if not ids:
            raise ValueError("empty prompt")
        fut = Future()
        with self._cv:
            if self._closed or self._error is not None:
                raise RuntimeError("engine server is closed") from self._error
            rid = self._next_id
            self._next_id += 1
            self._futures[rid] = fut
            if on_tokens is not None:
                self._callbacks[rid] = [on_tokens, 0]
            self._queue.append((rid, ids, min(int(max_tokens or self.max_new_tokens), self.max_new_tokens)))
            self._cv.notify_all()
        return fut

    def generate(self, prompt_token_ids, max_tokens: Optional[int] = None, timeout: Optional[float] = None, on_tokens=None):
        return self.submit(prompt_token_ids, max_tokens, on_tokens=on_tokens).result(timeout)

    @property
    def streaming(self) -> bool:
        """True while a request with a token callback is queued or running (the loop then reports progress)."""
        return bool(self._callbacks)

    def progress(self, rid, toks, lps) -> None:
        """Called by the engine loop with everything request `rid` has produced so far."""
        with self._cv:
            cb = self._callbacks.get(rid)
            if cb is None or len(toks) <= cb[1]:
                return
            fn, sent = cb
            cb[1] = len(toks)
        try:
            fn(np.array(toks[sent:], np.int64), np.array(lps[sent:], np.float32))
        except Exception:                          # a client's callback must not take the engine loop down
            import logging
            logging.getLogger(__name__).exception("token callback of request %s failed", rid)

    def pause(self, timeout: Optional[float] = None) -> bool:
        """Stop admitting requests and wait until the running ones are delivered. True when drained in time."""
        with self._cv:
            self._drained.clear()
            self._paused = True
            self._cv.notify_all()
        return self._drained.wait(timeout)

    def resume(self) -> None:
        with self._cv:
            self._paused = False
            self._cv.notify_all()

    def close(self, timeout: Optional[float] = 60.0) -> None:
        with self._cv:
            self._closed = True
            self._cv.notify_all()
        self._thread.join(timeout)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ------------------------------------------------------------------ request source of PagedEngine._loop
    def take(self, n_free):
        out = []
        with self._cv:
            while not self._paused and self._queue and len(out) < n_free:
                rid, ids, lim = self._queue.popleft()
                row = np.full(self.P, self.pad_id, np.int64)
                row[self.P - len(ids):] = ids
                out.append((rid, row, len(ids), lim))
            self.admitted += len(out)
        return out

    def give_back(self, items):
        with self._cv:
            for rid, row, ln, lim in reversed(items):
                self._queue.appendleft((rid, [int(t) for t in row[len(row) - ln:]], lim))
            self.admitted -= len(items)

    def more_waiting(self):
        with self._cv:
            return bool(self._queue) and not self._paused

    def deliver(self, rid, toks, lps):
        self.progress(rid, toks, lps)              # whatever has not been reported yet
        with self._cv:
            fut = self._futures.pop(rid)
            self._callbacks.pop(rid, None)
        fut.set_result((np.array(toks, np.int64), np.array(lps, np.float32)))

    def idle(self):
        refresh = False
        with self._cv:
            while True:
                if self._closed:
                    return False
                if self._paused:
                    self._drained.set()
                    refresh = True
                elif self._queue:
                    break
                self._cv.wait(0.05)
        if refresh:                                   # weights may have been updated while the server was paused
            self.engine._fuse_all()
            if self.engine._packed_on:
                self.engine._pack_all()
        return True

    def _serve(self):
        eng = self.engine
        try:
            if eng.device.type == "cuda":
                torch.cuda.set_device(eng.device)
            with torch.no_grad():
                eng._fuse_all()
                eng._packed_on = eng.pack_weights and eng.max_running <= 128
                if eng._packed_on:
                    eng._pack_all()
                t, p, k, seed = self._sampling
                st = eng._new_state(eng.max_running, self.max_new_tokens, self._eos, self.pad_id, t, p, k, seed)
                eng._loop(st, eng.max_running, self.max_new_tokens, self.pad_id, self)
        except BaseException as e:                    # hand the failure to every waiting client
            with self._cv:
                self._error = e
                self._closed = True
                futs = list(self._futures.values())
                self._futures.clear()
                self._callbacks.clear()
            for f in futs:
                f.set_exception(e)
            self._drained.set()
