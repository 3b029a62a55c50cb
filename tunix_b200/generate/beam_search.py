"""Batched beam search over the dense KV cache (tunix/generate/beam_search.py:39-305).

State per batch row: `beam_size` live hypotheses with cumulative log-probs; finished hypotheses (EOS) are
retained with their score and no longer expanded; the KV cache is gathered along the batch dim after each
step to follow the surviving beams. Returns the best hypothesis per row as [B, max_steps] token ids.
"""
from __future__ import annotations

import torch


@torch.no_grad()
def beam_search(model, prompts, plens, max_steps: int, beam_size: int, eos_ids, pad_id: int, dtype, device):
    B, P = prompts.shape
    K = beam_size
    toks = torch.from_numpy(prompts).to(device)
    lens = torch.from_numpy(plens).to(device)
    seg = (torch.arange(P, device=device)[None] >= (P - lens)[:, None]).to(torch.int32)
    positions = torch.clamp(torch.cumsum(seg, -1) - 1, min=0).to(torch.int32)
    # replicate every prompt K times: rows [b*K, (b+1)*K)
    rep = lambda t: t.repeat_interleave(K, dim=0)  # noqa: E731
    cache = model.init_cache(B * K, P + max_steps, dtype, device)
    hidden, cache = model(rep(toks), positions=rep(positions), cache=cache, segment_ids=rep(seg), skip_lm_head=True)
    next_pos = rep(positions[:, -1:]) + 1
    scores = torch.zeros(B, K, device=device)
    scores[:, 1:] = -1e30                       # only the first copy is live at step 0
    finished = torch.zeros(B, K, dtype=torch.bool, device=device)
    out = torch.full((B, K, max_steps), pad_id, dtype=torch.long, device=device)
    eos_t = torch.as_tensor(list(eos_ids), device=device)
    last_h = hidden[:, -1:]
    ones = torch.ones(B * K, 1, dtype=torch.int32, device=device)
    for step in range(max_steps):
        logits = model.compute_final_logits(last_h)[:, 0].float()
        logp = torch.log_softmax(logits, -1).view(B, K, -1)
        V = logp.shape[-1]
        # finished beams may only "emit" pad with zero cost so they compete on their final score
        keep = torch.full_like(logp, -1e30)
        keep[..., pad_id] = 0.0
        logp = torch.where(finished[..., None], keep, logp)
        cand = (scores[..., None] + logp).view(B, K * V)
        top_s, top_i = torch.topk(cand, K, dim=-1)
        src = top_i // V
        tok = top_i % V
        base = (torch.arange(B, device=device) * K)[:, None]
        flat_src = (base + src).view(-1)
        out = torch.gather(out, 1, src[..., None].expand(-1, -1, max_steps))
        was_finished = torch.gather(finished, 1, src)
        out[:, :, step] = torch.where(was_finished, torch.full_like(tok, pad_id), tok)
        finished = was_finished | (tok[..., None] == eos_t).any(-1)
        scores = top_s
        if bool(finished.all()):
            break
        for layer in cache:
            layer["k"] = layer["k"].index_select(0, flat_src)
            layer["v"] = layer["v"].index_select(0, flat_src)
            layer["seg"] = layer["seg"].index_select(0, flat_src)
        next_pos = next_pos.index_select(0, flat_src)
        hidden, cache = model(out[:, :, step].reshape(-1, 1), positions=next_pos, cache=cache, segment_ids=ones,
                              skip_lm_head=True)
        last_h = hidden
        next_pos = next_pos + 1
    best = scores.argmax(-1)
    return out[torch.arange(B, device=device), best]
