"""PagedEngine: the in-framework GPU rollout engine (paged KV cache, CUDA-graphed decode).

It takes the place of the reference's vLLM / SGLang-JAX integrations (tunix/generate/vllm_sampler.py,
sglang_jax_sampler.py) and follows the page-table conventions of its host-side paged-KV prototype
(tunix/experimental/generate/single_type_kv_cache_manager.py, tiered_page_pool.py): fixed-size pages, a
free list, one page table row per running sequence.

Per wave of at most `max_running_requests` sequences:
  prefill  one pass over the left-padded prompts with the tcgen05 flash-attention kernel; K / V of every
           layer are scattered into the pages by `kv_write` (padding is skipped);
  decode   every step is the same fixed sequence of kernel launches (embedding -> per layer RMSNorm, tcgen05
           GEMMs with narrow tiles, RoPE at device-resident positions, `kv_write`, `paged_decode` attention,
           GLU -> final norm -> lm_head GEMM in fp32 -> fused sampling kernel), all reading sequence lengths,
           the step counter and the page table from device memory, so the whole step is captured once in a
           CUDA graph and replayed; the host only checks every `check_every` steps whether all sequences hit EOS.
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
    """Device page pools for every layer plus the host-side free list."""

    def __init__(self, cfg, num_pages: int, page_size: int, max_seqs: int, max_pages_per_seq: int, device, dtype):
        self.page_size, self.num_pages, self.max_pages = page_size, num_pages, max_pages_per_seq
        row = cfg.num_kv_heads * cfg.head_dim
        # zero-initialised: rows of a page that were never written must hold finite values
        self.k = [torch.zeros(num_pages, page_size, row, dtype=dtype, device=device) for _ in range(cfg.num_layers)]
        self.v = [torch.zeros(num_pages, page_size, row, dtype=dtype, device=device) for _ in range(cfg.num_layers)]
        self.table_host = np.full((max_seqs, max_pages_per_seq), -1, np.int32)
        self.table = torch.full((max_seqs, max_pages_per_seq), -1, dtype=torch.int32, device=device)
        self._free = list(range(num_pages - 1, -1, -1))
        self._owned: dict = {}

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def reserve(self, slot: int, n_tokens: int) -> None:
        need = (n_tokens + self.page_size - 1) // self.page_size
        if need > self.max_pages:
            raise ValueError(f"sequence of {n_tokens} tokens needs {need} pages, table holds {self.max_pages}")
        have = self._owned.setdefault(slot, [])
        while len(have) < need:
            if not self._free:
                raise RuntimeError("out of KV pages")
            p = self._free.pop()
            self.table_host[slot, len(have)] = p
            have.append(p)

    def release(self, slot: int) -> None:
        pages = self._owned.pop(slot, [])
        if not pages:
            return
        for p in pages:
            if p in self._free:
                raise RuntimeError(f"double free of page {p}")
            self._free.append(p)
        self.table_host[slot, :] = -1

    def sync_table(self) -> None:
        self.table.copy_(torch.from_numpy(self.table_host), non_blocking=False)


class PagedEngine(BaseSampler):
    def __init__(self, transformer, tokenizer, cache_config: CacheConfig, page_size: int = 64,
                 max_running_requests: int = 64, use_cuda_graph: bool = True, check_every: int = 16,
                 use_pdl: bool = False, pack_weights: bool = True):
        self._model = transformer
        self.tokenizer = tokenizer
        self.cfg = transformer.config
        self.cache_size = cache_config.cache_size
        self.device = next(transformer.parameters()).device
        self.dtype = next(transformer.parameters()).dtype
        if self.device.type != "cuda" or self.dtype != torch.bfloat16:
            raise ValueError("PagedEngine runs bf16 models on CUDA; use Sampler elsewhere")
        if self.cfg.is_moe:
            raise NotImplementedError("MoE decode goes through Sampler")
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
        self._packed = None
        self.check_every = check_every
        self.max_pages_per_seq = (self.cache_size + page_size - 1) // page_size
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
            pages = self.max_running * self.max_pages_per_seq
            self.pool = PagePool(self.cfg, pages, self.page_size, self.max_running, self.max_pages_per_seq, self.device,
                                 self.dtype)

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
            self._wgu.append(self._fused_weight([layer.mlp.gate_proj, layer.mlp.up_proj]))

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
            srcs.append({"qkv": self._wqkv[i], "o": at.o_proj.weight.data if self._plain(at.o_proj) else None,
                         "gu": self._wgu[i], "down": mlp.down_proj.weight.data if self._plain(mlp.down_proj) else None})
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
            self._packed = [{name: (K.PackedWeight(w) if w is not None else None) for name, w in src.items()} for src in srcs]
            self._graph = None          # a captured graph points at the old buffers
            return
        for have, src in zip(self._packed, srcs):
            for name, w in src.items():
                if have[name] is not None:
                    have[name].refresh(w)

    def _pk(self, i, name):
        return self._packed[i].get(name) if self._packed is not None else None

    def _rope(self, i):
        return self._model._rope(self.cfg.layer_type(i) == "local", self.device)

    def _attn_in(self, layer, h2, positions_flat, i):
        """Projections + QK-norm + RoPE on flat rows h2 [n, D] -> q [n,N,H], k [n,K,H], v [n,K*H]."""
        cfg, at = self.cfg, layer.self_attn
        N, KH, H = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
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
        if wgu is None:
            return layer.mlp(h, residual=residual)
        Fd = wgu.shape[0] // 2
        h2 = h.reshape(-1, h.shape[-1])
        pgu = self._pk(i, "gu") if decode else None
        gu = K.gemm_packed(h2, pgu) if pgu is not None else F.linear(h2, wgu)
        a = K.glu_fwd(gu[:, :Fd], gu[:, Fd:], K.GLU_SILU if layer.mlp.kind == "silu" else K.GLU_GELU)
        pdown = self._pk(i, "down") if decode else None
        if pdown is not None:
            r2 = residual.reshape(-1, residual.shape[-1]) if residual is not None else None
            return K.gemm_packed(a, pdown, residual=r2).view(*h.shape[:-1], -1)
        return layer.mlp.down_proj(a.view(*h.shape[:-1], Fd), residual=residual)

    def _mlp_and_norms(self, layer, i, x, attn_out, decode=False):
        cfg = self.cfg
        if cfg.post_norms:
            x = x + layer.post_attn_norm(attn_out)
            m = self._mlp(layer, i, layer.post_attention_layernorm(x), decode=decode)
            return x + layer.post_ffw_norm(m)
        x = attn_out          # o_proj already added the residual
        return self._mlp(layer, i, layer.post_attention_layernorm(x), residual=x, decode=decode)

    def _prefill(self, toks, positions, seg, slots):
        """toks [B,P] left padded. Writes K/V pages, returns hidden state of the last position [B, D]."""
        cfg, pool = self.cfg, self.pool
        B, P = toks.shape
        x = F.embedding(toks, self._model.embed_tokens, math.sqrt(cfg.embed_dim) if cfg.embed_scale else 1.0)
        pos_flat = positions.reshape(-1).contiguous()
        wpos = torch.where(seg.reshape(-1) > 0, pos_flat, torch.full_like(pos_flat, -1))
        seq_ids = slots.repeat_interleave(P)
        for i, layer in enumerate(self._model.layers):
            h = layer.input_layernorm(x)
            q, k, v = self._attn_in(layer, h.view(B * P, -1), pos_flat, i)
            K.kv_write(k.view(B * P, -1), v, seq_ids, wpos, pool.table, pool.page_size, pool.k[i], pool.v[i])
            at = layer.self_attn
            o = F.attention(q.view(B, P, cfg.num_heads, cfg.head_dim), k.view(B, P, cfg.num_kv_heads, cfg.head_dim),
                            v.view(B, P, cfg.num_kv_heads, cfg.head_dim), scale=at.scale, causal=True, window=at.window,
                            softcap=cfg.attn_logit_softcap, seg_q=seg, seg_k=seg)
            o = o.reshape(B, P, -1)
            a = at.o_proj(o, residual=None if cfg.post_norms else x)
            x = self._mlp_and_norms(layer, i, x, a)
        return self._model.norm(x[:, -1])

    def _decode_step(self, st) -> None:
        """One token for every sequence of the wave. `st` holds the static device buffers."""
        cfg, pool = self.cfg, self.pool
        B = st["tokens"].shape[0]
        N, KH, H = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
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
                               softcap=cfg.attn_logit_softcap, window=at.window, workspace=st["ws"])
            po = self._pk(i, "o")
            if po is not None:
                a = K.gemm_packed(o.view(B, N * H), po, residual=None if cfg.post_norms else x)
            else:
                a = at.o_proj(o.view(B, N * H), residual=None if cfg.post_norms else x)
            x = self._mlp_and_norms(layer, i, x, a, decode=True)
        hlast = self._model.norm(x)
        self._sample_into(hlast, st, advance=True)

    def _sample_into(self, hlast, st, advance: bool) -> None:
        ph = self._pk(len(self._model.layers), "head")
        if ph is not None:
            logits = K.gemm_packed(hlast, ph, out=st["logits"])
        else:
            logits = K.gemm(hlast, self._model.head_weight(), out=st["logits"])
        if self.cfg.final_logit_softcap:
            c = self.cfg.final_logit_softcap
            logits.copy_(c * torch.tanh(logits / c))
        p = st["params"]
        S.sample(logits, p["temperature"], p["top_p"], p["top_k"], p["seed"], 0, want_logprob=True,
                 out_tokens=st["next"], out_logprobs=st["next_lp"], step_tensor=st["step"])
        done = st["done"]
        tok = torch.where(done, st["pad"], st["next"])
        idx = st["step"].to(torch.int64).view(1, 1).expand(tok.shape[0], 1)
        st["out_tokens"].scatter_(1, idx, tok[:, None])
        st["out_lp"].scatter_(1, idx, torch.where(done, torch.zeros_like(st["next_lp"]), st["next_lp"])[:, None])
        st["done"].copy_(done | (tok[:, None] == st["eos"]).any(-1))
        # the sampled token is fed at the next decode step; a decode step also moves the write position on
        st["tokens"].copy_(tok)
        if advance:
            st["positions"].copy_(st["seq_lens"])
            st["seq_lens"].add_(1)
        st["step"].add_(1)

    # --------------------------------------------------------------------- call
    @torch.no_grad()
    def __call__(self, input_strings=None, max_generation_steps: int = 0, max_prompt_length: Optional[int] = None,
                 echo: bool = False, return_logits: bool = False, return_logprobs: bool = False,
                 eos_tokens: Optional[Sequence[int]] = None, forbidden_tokens=None, temperature: float = 0.0,
                 top_p: Optional[float] = None, top_k: Optional[int] = None, beam_size=None, seed: Optional[int] = None,
                 pad_output: bool = False, *, prompt_token_ids=None) -> SamplerOutput:
        if forbidden_tokens or beam_size or return_logits or echo:
            raise NotImplementedError("forbidden tokens, beam search, logits and echo are served by Sampler")
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
        all_tokens, all_lps = [], []
        prompts_all, plens_all = pad_prompts_left(rows, plen, pad_id)
        self._fuse_all()
        self._pack_all()
        for w0 in range(0, len(rows), self.max_running):
            toks_np, lens_np = prompts_all[w0:w0 + self.max_running], plens_all[w0:w0 + self.max_running]
            gen, lps = self._run_wave(toks_np, lens_np, max_generation_steps, eos_ids, pad_id, temperature, top_p, top_k,
                                      (seed or 0) + w0)
            all_tokens.append(gen)
            all_lps.append(lps)
        self._model.train(was_training)
        gen = np.concatenate(all_tokens)
        lps = np.concatenate(all_lps)
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

    def _run_wave(self, toks_np, lens_np, max_steps, eos_ids, pad_id, temperature, top_p, top_k, seed):
        dev = self.device
        B, P = toks_np.shape
        self._ensure_pool(B)
        self._fuse_all()
        pool = self.pool
        for s in range(B):
            pool.release(s)
            pool.reserve(s, int(lens_np[s]) + max_steps + 1)
        pool.sync_table()
        toks = torch.from_numpy(toks_np).to(dev)
        lens = torch.from_numpy(lens_np).to(dev)
        seg = (torch.arange(P, device=dev)[None] >= (P - lens)[:, None]).to(torch.int32)
        positions = torch.clamp(torch.cumsum(seg, -1) - 1, min=0).to(torch.int32)
        slots = torch.arange(B, device=dev, dtype=torch.int32)
        hlast = self._prefill(toks, positions, seg, slots)
        splits = (self.cache_size + K.DECODE_SPLIT_TOKENS - 1) // K.DECODE_SPLIT_TOKENS
        N, H, V = self.cfg.num_heads, self.cfg.head_dim, self.cfg.vocab_size
        st = {
            "tokens": torch.zeros(B, dtype=torch.int64, device=dev),
            "positions": lens.to(torch.int32).clone(),            # first generated token sits at position len
            "seq_lens": (lens + 1).to(torch.int32),
            "slots": slots, "done": torch.zeros(B, dtype=torch.bool, device=dev),
            "next": torch.zeros(B, dtype=torch.int64, device=dev), "next_lp": torch.zeros(B, device=dev),
            "out_tokens": torch.full((B, max(max_steps, 1)), pad_id, dtype=torch.int64, device=dev),
            "out_lp": torch.zeros((B, max(max_steps, 1)), device=dev),
            "logits": torch.empty(B, V, dtype=torch.float32, device=dev),
            "step": torch.zeros(1, dtype=torch.int32, device=dev),
            "pad": torch.full((B,), pad_id, dtype=torch.int64, device=dev),
            "eos": torch.as_tensor(eos_ids, device=dev, dtype=torch.int64),
            "ws": (torch.empty(B * N * splits * H, dtype=torch.float32, device=dev),
                   torch.empty(B * N * splits * 2, dtype=torch.float32, device=dev)),
            "params": {"temperature": temperature, "top_p": top_p, "top_k": top_k, "seed": seed},
        }
        if max_steps == 0:
            return st["out_tokens"][:, :0].cpu().numpy(), st["out_lp"][:, :0].cpu().numpy()
        # token 0 comes from the prefill's last hidden state; it will sit at position `len`
        self._sample_into(hlast, st, advance=False)
        from .. import _lib
        _lib.register_cuda_sigs({"tb_set_pdl": [_lib.I]})
        _lib.cuda().tb_set_pdl(1 if self.use_pdl else 0)
        try:
            return self._decode_loop(st, max_steps, pool, B)
        finally:
            _lib.cuda().tb_set_pdl(0)

    def _decode_loop(self, st, max_steps, pool, B):
        graph = None
        if self.use_graph and max_steps > 2:
            # warm the decode path once outside capture (lazy kernel attribute setup, tensor-map cache), then
            # capture one step and replay it
            snap = {k: st[k].clone() for k in ("tokens", "positions", "seq_lens", "done", "out_tokens", "out_lp", "step")}
            self._decode_step(st)
            for k, v in snap.items():
                st[k].copy_(v)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._decode_step(st)
            for k, v in snap.items():
                st[k].copy_(v)
        for step in range(1, max_steps):
            if graph is not None:
                graph.replay()
            else:
                self._decode_step(st)
            if step % self.check_every == 0 and bool(st["done"].all()):
                break
        for s in range(B):
            pool.release(s)
        return st["out_tokens"].cpu().numpy(), st["out_lp"].cpu().numpy()
