"""Data-parallel training with sharded optimizer state: fused reduce-scatter + AdamW over NVLink.

What the reference gets from GSPMD for its `fsdp` mesh axis (per-use parameter all-gather, gradient
reduce-scatter, optimizer state sharded like the parameters; tunix/models/llama3/model.py:65-82,
tunix/sft/peft_trainer.py:609-650) is done here explicitly, sized for 180 GB of HBM per GPU:

* the bf16 working copy of the model stays resident and replicated (16 GB for an 8B model), so weights
  cross NVLink once per optimizer step instead of once per use;
* fp32 master weights and Adam moments are sharded 1/W per rank (per tensor, along dim 0);
* gradients are written by the wgrad GEMMs straight into a flat buffer in symmetric memory. When the
  backward pass leaves a decoder layer, that layer's bucket is reduced on a side stream while backward
  continues: a flag barrier (bounded wait), then ONE kernel that pulls the rank's slice of every peer's
  gradients over NVLink, sums in fp32, applies the 1/denominator scale, writes the fp32 shard and
  accumulates its sum of squares for the global grad-norm (csrc/comm.cu);
* after a scalar all-reduce of the squared norm, ONE AdamW kernel updates the shard (clip factor read
  from device memory) and emits the bf16 shard into symmetric memory; an all-gather kernel then pulls
  every peer's updated shard into the resident bf16 copy.

`comm="nccl"` runs the same schedule on NCCL collectives (all-reduce + all-gather): the in-repo baseline
the fused path is measured against. With world size 1 (or on CPU ranks under gloo) it degrades to the
plain flat-buffer AdamW.
"""
from __future__ import annotations

import ctypes
import re
from typing import Iterable, Optional

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn

from .. import _lib
from ..optim import AdamW, Optimizer, install_grad_fold_hook
from . import symm

P, LL, I, F = _lib.P, _lib.LL, _lib.I, _lib.F
_lib.register_cuda_sigs({
    "tb_reduce_scatter_pull": [P, I, P, I, I, I, P, F, P, I, P],
    "tb_allgather_pull": [P, P, I, I, I, P, I, P],
    "tb_gather_shard": [P, P, I, I, P, P, P],
})

CHUNK_ELEMS = 1 << 16
_CHUNK_DT = np.dtype([("full_off", "<i8"), ("shard_off", "<i8"), ("rank_stride", "<i8"), ("len", "<i4"),
                      ("pad", "<i4")])


def _bucket_of(name: str, num_layers_hint: int = 0) -> int:
    """-1: embeddings (ready last in backward); i: decoder layer i; 10**6: final norm / lm_head (ready first)."""
    m = re.search(r"layers\.(\d+)\.", name)
    if m:
        return int(m.group(1))
    if "embed" in name:
        return -1
    return 10 ** 6


class ShardedAdamW(AdamW):
    is_sharded = True

    def __init__(self, learning_rate=1e-3, b1=0.9, b2=0.999, eps=1e-8, weight_decay=1e-4, max_grad_norm=None,
                 group=None, comm: str = "p2p", overlap: bool = True, barrier_timeout_ms: int = 30000,
                 defer_gather: bool = False, gather_ctas: int = 64):
        super().__init__(learning_rate, b1, b2, eps, weight_decay, max_grad_norm)
        self.group, self.comm, self.overlap = group, comm, overlap
        # tuning overrides for measurements: TUNIX_B200_FSDP_DEFER=0/1, TUNIX_B200_FSDP_GATHER_CTAS=n
        import os
        env = os.environ.get
        self.defer_gather = bool(int(env("TUNIX_B200_FSDP_DEFER", "1" if defer_gather else "0")))
        self.gather_ctas = int(env("TUNIX_B200_FSDP_GATHER_CTAS", str(gather_ctas)))
        # "dma": the overlapped all-gather runs on the copy engines; "kernel": on `gather_ctas` CTAs of the pull kernel
        self.gather_engine = env("TUNIX_B200_FSDP_GATHER", "dma")
        self.barrier_timeout_ms = barrier_timeout_ms
        self._update_pending = True
        self._reduced: set = set()
        self.comm_launches = 0

    # ------------------------------------------------------------------- bind
    def bind(self, named_params: Iterable[tuple[str, nn.Parameter]], grad_dtype=None, pad_to_multiple: int = 1):
        named = list(named_params)
        self.world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        dev = named[0][1].device
        if self.world == 1 or dev.type != "cuda":
            self.is_sharded = self.world > 1
            if self.world == 1:
                return super().bind(named, grad_dtype, pad_to_multiple)
        W = self.world
        dt = named[0][1].dtype
        assert dt == torch.bfloat16 or dev.type != "cuda", "sharded GPU training expects bf16 parameters"
        self.names = [n for n, _ in named]
        self.params = [p for _, p in named]
        unit = 8 * W
        self.offsets, self.lens, off = [], [], 0
        for p in self.params:
            ln = (p.numel() + unit - 1) // unit * unit
            self.offsets.append(off)
            self.lens.append(ln)
            off += ln
        self.total = off
        self.shard_total = off // W
        self.grad_dtype = grad_dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32)
        use_symm = dev.type == "cuda" and self.comm == "p2p" and symm.symm_available(self.group)
        if dev.type == "cuda" and self.comm == "p2p" and not use_symm:
            raise RuntimeError("comm='p2p' needs torch symmetric memory over NCCL; pass comm='nccl' for the baseline path")
        self.param_flat = torch.zeros(self.total, dtype=dt, device=dev)
        if use_symm:
            self.grad_buf = symm.symm_empty(self.total, self.grad_dtype, dev, self.group)
            self.shard16_buf = symm.symm_empty(self.shard_total, dt, dev, self.group)
            self.barrier = symm.SymmBarrier(dev, self.group, self.barrier_timeout_ms)
        else:
            self.grad_buf = symm.SymmBuffer(torch.zeros(self.total, dtype=self.grad_dtype, device=dev), [0], 0, 1)
            self.shard16_buf = symm.SymmBuffer(torch.zeros(self.shard_total, dtype=dt, device=dev), [0], 0, 1)
            self.barrier = None
        self.grad_flat = self.grad_buf.tensor
        self.shard16 = self.shard16_buf.tensor
        with torch.no_grad():
            for p, o in zip(self.params, self.offsets):
                view = self.param_flat[o:o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.main_grad = self.grad_flat[o:o + p.numel()].view(p.shape)
                p.grad_added_to_main_grad = False
                install_grad_fold_hook(p)
        # shard-local state
        self.master = torch.zeros(self.shard_total, dtype=torch.float32, device=dev)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.red32 = torch.zeros_like(self.master)
        self._stats = torch.zeros(2, dtype=torch.float32, device=dev)   # [sum g^2 of the shard, denominator]
        self._sumsq = self._stats[:1]
        self._param_events: dict = {}
        # chunk tables per bucket
        self.shard_offsets, soff = [], 0
        for ln in self.lens:
            self.shard_offsets.append(soff)
            soff += ln // W
        buckets: dict = {}
        for i, n in enumerate(self.names):
            buckets.setdefault(_bucket_of(n), []).append(i)
        self.bucket_tables: dict = {}
        for b, idxs in buckets.items():
            rows = []
            for i in idxs:
                stride = self.lens[i] // W
                for t0 in range(0, stride, CHUNK_ELEMS):
                    rows.append((self.offsets[i] + t0, self.shard_offsets[i] + t0, stride,
                                 min(CHUNK_ELEMS, stride - t0), 0))
            arr = np.array(rows, dtype=_CHUNK_DT)
            tab = torch.from_numpy(arr.view(np.uint8).copy()).to(dev)
            self.bucket_tables[b] = (tab, len(rows))
        self.bucket_order = sorted(self.bucket_tables, reverse=True)  # order in which backward completes them
        self._native_dev = dev.type == "cuda"
        self.comm_stream = torch.cuda.Stream(device=dev) if (self._native_dev and self.overlap) else None
        # Views for checkpointing / state_dict in terms of the full parameter tensors are gathered on demand.
        self.buffers = _ShardedBuffersFacade(self)
        self._init_master()
        return self

    def _init_master(self) -> None:
        if self._native_dev:
            lib = _lib.cuda()
            for b, (tab, n) in self.bucket_tables.items():
                _lib.check(lib.tb_gather_shard(self.param_flat.data_ptr(), tab.data_ptr(), n, self.rank,
                                               self.master.data_ptr(), self.shard16.data_ptr(), _lib.stream_ptr()),
                           "tb_gather_shard")
        else:
            for i in range(len(self.params)):
                s = self.lens[i] // self.world
                src = self.param_flat[self.offsets[i] + self.rank * s: self.offsets[i] + (self.rank + 1) * s]
                self.master[self.shard_offsets[i]:self.shard_offsets[i] + s] = src.float()

    # -------------------------------------------------------------- backward
    def prepare_backward(self, is_update_step: bool) -> None:
        self._update_pending = is_update_step
        if is_update_step and self.is_sharded and getattr(self, "params", None) is not None:
            # the flags now tell which gradients of THIS backward pass have reached the flat buffer
            for p in self.params:
                p.grad_added_to_main_grad = False

    def install_hooks(self, model) -> None:
        """Ask the model to report when backward leaves each decoder layer (see Transformer.layer_grad_hook)."""
        model.layer_grad_hook = self.on_layer_backward_done
        if not (self.is_sharded and getattr(self, "_native_dev", False) and self.comm_stream is not None
                and self.comm == "p2p" and self.defer_gather):
            return
        # the parameter pulls of the last update may still be in flight when the next forward starts: every
        # part of the model waits for its own bucket, anything unrecognised waits for all of them
        layers = getattr(model, "layers", None)
        if layers is None or type(model).__name__ != "Transformer" or getattr(model, "tp", None) is not None:
            # other model classes read parameters outside the embed -> layers -> norm -> head order this relies on
            self.defer_gather = False
            return
        model.register_forward_pre_hook(lambda m, a: self.wait_bucket(-1))
        for i, layer in enumerate(layers):
            layer.register_forward_pre_hook(lambda m, a, i=i: self.wait_bucket(i))
        known = set(range(len(layers))) | {-1, 10 ** 6}
        if not set(self.bucket_tables) <= known:
            self.defer_gather = False
        self._tail_hooks(model)

    def _tail_hooks(self, model) -> None:
        tail = lambda *a, **k: self.wait_bucket(10 ** 6)  # noqa: E731
        norm = getattr(model, "norm", None)
        if norm is not None:
            norm.register_forward_pre_hook(tail)
        else:
            self.defer_gather = False

    def on_layer_backward_done(self, layer_idx: int) -> None:
        """Called from autograd when all gradients of buckets > layer_idx .. are complete.

        Boundary `i` sits at the input of decoder layer i, boundary L at the output of the last layer."""
        if not (self.is_sharded and self._update_pending and self.overlap and self._native_dev):
            return
        ready = [b for b in self.bucket_order if b >= layer_idx and b not in self._reduced
                 and self._bucket_complete(b)]
        if ready:
            self._reduce_buckets(ready)

    def _bucket_complete(self, b: int) -> bool:
        """A bucket may be reduced during backward only if every trainable tensor in it has already put this pass's
        gradient into the flat buffer. Gradients that autograd delivers through `.grad` (ops without a
        `main_grad` epilogue) are folded in here when they have arrived; a bucket still missing one waits for
        `step()`, which reduces it after `collect_autograd_grads()`."""
        for i in self._bucket_param_idx_cached(b):
            p = self.params[i]
            if not p.requires_grad:
                continue
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(self.grad_dtype))
                p.grad = None
                p.grad_added_to_main_grad = True
            if not getattr(p, "grad_added_to_main_grad", False):
                return False
        return True

    def _bucket_param_idx_cached(self, b: int) -> list:
        cache = getattr(self, "_bucket_idx", None)
        if cache is None:
            cache = self._bucket_idx = {}
        if b not in cache:
            cache[b] = self._bucket_param_idx(b)
        return cache[b]

    def _reduce_buckets(self, buckets: list) -> None:
        lib = _lib.cuda()
        main = torch.cuda.current_stream()
        stream = self.comm_stream or main
        if stream is not main:
            ev = torch.cuda.Event()
            ev.record(main)
            stream.wait_event(ev)
        with torch.cuda.stream(stream):
            if self.comm == "nccl":
                for b in buckets:
                    idx = self._bucket_param_idx(b)  # a bucket's tensors are adjacent in the flat buffer
                    lo = min(self.offsets[i] for i in idx)
                    hi = max(self.offsets[i] + self.lens[i] for i in idx)
                    dist.all_reduce(self.grad_flat[lo:hi], group=self.group)
            else:
                self.barrier.wait(slot=0)
                self.comm_launches += 1
            for b in buckets:
                tab, n = self.bucket_tables[b]
                if self.comm == "nccl":
                    # grads are already summed everywhere: pick this rank's slice with a 1-rank "pull"
                    local = (ctypes.c_void_p * 8)(self.grad_flat.data_ptr() + 0, *([None] * 7))
                    rc = lib.tb_reduce_scatter_pull(ctypes.cast(local, ctypes.c_void_p),
                                                    1 if self.grad_dtype == torch.bfloat16 else 0,
                                                    self._rank_shifted_table(b).data_ptr(), n, 0, 1,
                                                    self.red32.data_ptr(), 1.0, self._sumsq.data_ptr(), 0,
                                                    stream.cuda_stream)
                else:
                    rc = lib.tb_reduce_scatter_pull(self.grad_buf.c_ptrs, 1 if self.grad_dtype == torch.bfloat16 else 0,
                                                    tab.data_ptr(), n, self.rank, self.world, self.red32.data_ptr(),
                                                    1.0, self._sumsq.data_ptr(), 32 if self.overlap else 0,
                                                    stream.cuda_stream)
                _lib.check(rc, "tb_reduce_scatter_pull")
                self.comm_launches += 1
                self._reduced.add(b)

    def _bucket_param_idx(self, b: int) -> list:
        return [i for i, n in enumerate(self.names) if _bucket_of(n) == b]

    def _rank_shifted_table(self, b: int) -> torch.Tensor:
        """Chunk table whose full offsets already include this rank's piece (for 1-rank kernels)."""
        cache = getattr(self, "_shifted", None)
        if cache is None:
            cache = self._shifted = {}
        if b not in cache:
            tab, n = self.bucket_tables[b]
            arr = tab.cpu().numpy().view(_CHUNK_DT).copy()
            arr["full_off"] += self.rank * arr["rank_stride"]
            cache[b] = torch.from_numpy(arr.view(np.uint8).copy()).to(tab.device)
        return cache[b]

    # ------------------------------------------------------------------ step
    def collect_autograd_grads(self) -> None:
        for p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(self.grad_dtype))
                p.grad = None

    def zero_grad(self) -> None:
        if not self.is_sharded or self.world == 1:
            return super().zero_grad()
        # peers finished reading these gradients before the barrier that follows the update completed, and the
        # current stream already waits for that barrier (see _gather_params)
        self.grad_flat.zero_()
        for p in self.params:
            p.grad = None

    reduces_denominator = True   # step(..., denominator_is_local=True) sums the ranks' denominators itself

    def step(self, denominator=1.0, sumsq: Optional[torch.Tensor] = None,
             denominator_is_local: bool = False) -> torch.Tensor:
        """One sharded update. `denominator` is a float, or a one-element device tensor that the host never reads;
        with `denominator_is_local` it is this rank's part and is summed over the group in the same all-reduce as
        the squared gradient norm."""
        if self.world == 1:
            return super().step(denominator, sumsq)
        if not self._native_dev:
            return self._step_cpu(denominator, denominator_is_local)
        lib = _lib.cuda()
        self.collect_autograd_grads()
        rest = [b for b in self.bucket_order if b not in self._reduced]
        if rest:
            self._reduce_buckets(rest)
        main = torch.cuda.current_stream()
        if self.comm_stream is not None:
            # also orders this update after the previous step's parameter pulls and its closing barrier
            main.wait_stream(self.comm_stream)
        self._param_events = {}
        den = self._stats[1:2]
        if isinstance(denominator, torch.Tensor):
            den.copy_(denominator.reshape(1).to(torch.float32))
        else:
            den.fill_(float(denominator))
        if denominator_is_local:
            dist.all_reduce(self._stats, group=self.group)      # [sum g^2, sum of denominators] in one message
        else:
            dist.all_reduce(self._sumsq, group=self.group)
        den.clamp_(min=1e-8)
        self.step_count += 1
        lr = self.learning_rate_at(self.step_count - 1)
        from ..ops import kernels as K
        K.adamw(self.master, self.m, self.v, self.red32, self.shard16, lr=lr, beta1=self.b1, beta2=self.b2,
                eps=self.eps, weight_decay=self.weight_decay, step=self.step_count, grad_scale=1.0,
                max_norm=self.max_grad_norm or 0.0, sumsq_buf=self._sumsq, denom_buf=den)
        grad_norm = self._sumsq.sqrt() / den
        if self.comm == "nccl":
            gathered = torch.empty(self.world * self.shard_total, dtype=self.shard16.dtype, device=self.shard16.device)
            dist.all_gather_into_tensor(gathered, self.shard16, group=self.group)
            ptr_arr = (ctypes.c_void_p * 8)(*[gathered.data_ptr() + r * self.shard_total * 2 for r in range(self.world)],
                                            *([None] * (8 - self.world)))
            shard_ptrs = ctypes.cast(ptr_arr, ctypes.c_void_p)
            for b in self.bucket_order:
                tab, n = self.bucket_tables[b]
                _lib.check(lib.tb_allgather_pull(shard_ptrs, tab.data_ptr(), n, self.rank, self.world,
                                                 self.param_flat.data_ptr(), 0, _lib.stream_ptr()), "tb_allgather_pull")
                self.comm_launches += 1
        else:
            self._gather_params(main)
        self._reduced.clear()
        self._stats.zero_()
        return grad_norm

    def _gather_params(self, main) -> None:
        """Pull every peer's updated bf16 shard into the resident copy, bucket by bucket in the order the next
        forward pass uses them. With `overlap` the pulls run on the side stream and the next forward waits per
        layer (`wait_bucket`), so only the first bucket's transfer is exposed; otherwise they run in line."""
        lib = _lib.cuda()
        deferred = self.comm_stream is not None and self.defer_gather
        stream = self.comm_stream if deferred else main
        if deferred:
            ev = torch.cuda.Event()
            ev.record(main)
            stream.wait_event(ev)
        with torch.cuda.stream(stream):
            # every rank's bf16 shard is final and every rank is done reading gradients once this barrier passes
            self.barrier.wait(slot=1)
            if deferred:
                grads_free = torch.cuda.Event()
                grads_free.record(stream)
            for b in sorted(self.bucket_tables):         # -1 (embeddings), layers 0..L-1, then the head
                if deferred and self.gather_engine == "dma":
                    # copy engines move the pieces (one peer-to-peer copy per tensor and peer): no SM is taken
                    # from the forward pass that runs meanwhile
                    for dst, src in self._dma_plan(b):
                        dst.copy_(src, non_blocking=True)
                        self.comm_launches += 1
                else:
                    tab, n = self.bucket_tables[b]
                    _lib.check(lib.tb_allgather_pull(self.shard16_buf.c_ptrs, tab.data_ptr(), n, self.rank, self.world,
                                                     self.param_flat.data_ptr(), self.gather_ctas if deferred else 0,
                                                     stream.cuda_stream), "tb_allgather_pull")
                    self.comm_launches += 1
                if deferred:
                    e = torch.cuda.Event()
                    e.record(stream)
                    self._param_events[b] = e
            # peers must finish pulling this rank's shard before the next update overwrites it: holds once
            # everyone passed this point (the next update waits for this stream)
            self.barrier.wait(slot=2)
        if deferred:
            main.wait_event(grads_free)      # the gradient buffer may be zeroed from here on

    def _dma_plan(self, b: int) -> list:
        """[(destination view in the resident parameters, source view in a peer's bf16 shard)] of bucket `b`."""
        plans = getattr(self, "_dma_plans", None)
        if plans is None:
            plans = self._dma_plans = {}
        if b not in plans:
            W, out = self.world, []
            peers = [self.shard16_buf.peer_tensor(p) for p in range(W)]
            for i in self._bucket_param_idx_cached(b):
                s_ = self.lens[i] // W
                for k in range(W):
                    p = (self.rank + 1 + k) % W                      # peers first, own piece last
                    src = peers[p][self.shard_offsets[i]:self.shard_offsets[i] + s_]
                    dst = self.param_flat[self.offsets[i] + p * s_: self.offsets[i] + (p + 1) * s_]
                    out.append((dst, src))
            plans[b] = out
        return plans[b]

    def wait_bucket(self, b: int) -> None:
        """Make the current stream wait until bucket `b` of the parameters holds the latest update."""
        ev = self._param_events.pop(b, None) if self._param_events else None
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def wait_params(self) -> None:
        """Make the current stream wait for every outstanding parameter pull (evaluation, checkpoints, weight
        sync and anything else that reads parameters outside the layer-by-layer forward)."""
        if self._param_events:
            self._param_events = {}
            torch.cuda.current_stream().wait_stream(self.comm_stream)

    def _step_cpu(self, denominator, denominator_is_local: bool = False) -> torch.Tensor:
        """gloo ranks: all-reduce gradients, update the local shard with the same math, all-gather."""
        self.collect_autograd_grads()
        g = self.grad_flat.float()
        dist.all_reduce(g, group=self.group)
        if denominator_is_local:
            d = torch.as_tensor(denominator, dtype=torch.float32).reshape(1).clone()
            dist.all_reduce(d, group=self.group)
            denominator = float(d)
        inv = 1.0 / max(float(denominator), 1e-8)
        W, r = self.world, self.rank
        shard_g = torch.cat([g[o + r * (ln // W): o + (r + 1) * (ln // W)] for o, ln in zip(self.offsets, self.lens)])
        sumsq = shard_g.pow(2).sum()
        dist.all_reduce(sumsq, group=self.group)
        self.step_count += 1
        t = self.step_count
        lr = self.learning_rate_at(t - 1)
        scale = inv
        if self.max_grad_norm:
            norm = float(sumsq.sqrt()) * inv
            scale *= self.max_grad_norm / max(norm, self.max_grad_norm)
        gs = shard_g * scale
        self.m.mul_(self.b1).add_(gs, alpha=1 - self.b1)
        self.v.mul_(self.b2).addcmul_(gs, gs, value=1 - self.b2)
        upd = (self.m / (1 - self.b1 ** t)) / ((self.v / (1 - self.b2 ** t)).sqrt() + self.eps)
        self.master.sub_(lr * (upd + self.weight_decay * self.master))
        shards = [torch.empty_like(self.master) for _ in range(W)]
        dist.all_gather(shards, self.master, group=self.group)
        with torch.no_grad():
            for i, (o, ln) in enumerate(zip(self.offsets, self.lens)):
                s = ln // W
                for p_ in range(W):
                    self.param_flat[o + p_ * s: o + (p_ + 1) * s] = shards[p_][self.shard_offsets[i]:self.shard_offsets[i] + s].to(self.param_flat.dtype)
        return sumsq.sqrt() * inv

    # ------------------------------------------------------------ checkpoints
    def state_dict(self) -> dict:
        """Full (unsharded) optimizer state, gathered over the group, keyed like the single-process optimizer."""
        if self.world == 1:
            return super().state_dict()
        out = {"step": self.step_count}
        for key, shard in (("mu", self.m), ("nu", self.v), ("master", self.master)):
            gathered = [torch.empty_like(shard) for _ in range(self.world)]
            dist.all_gather(gathered, shard, group=self.group)
            d = {}
            for i, (n, p) in enumerate(zip(self.names, self.params)):
                s = self.lens[i] // self.world
                full = torch.cat([g[self.shard_offsets[i]:self.shard_offsets[i] + s] for g in gathered])
                d[n] = full[:p.numel()].view(p.shape)
            out[key] = d
        return out

    def load_state_dict(self, sd: dict) -> None:
        if self.world == 1:
            return super().load_state_dict(sd)
        self.step_count = int(sd.get("step", 0))
        for key, shard in (("mu", self.m), ("nu", self.v), ("master", self.master)):
            if key not in sd:
                continue
            for i, n in enumerate(self.names):
                if n not in sd[key]:
                    continue
                s = self.lens[i] // self.world
                full = torch.zeros(self.lens[i], dtype=torch.float32)
                src = torch.as_tensor(sd[key][n]).reshape(-1).float()
                full[:src.numel()] = src
                shard[self.shard_offsets[i]:self.shard_offsets[i] + s] = full[self.rank * s:(self.rank + 1) * s].to(shard.device)

    def sync_master_from_params(self) -> None:
        if self.world == 1:
            return super().sync_master_from_params()
        self._init_master()

    def _state_tensors(self) -> dict:
        if self.world == 1:
            return super()._state_tensors()
        return {"mu": self.m, "nu": self.v, "master": self.master}


def shard_optimizer(opt: Optimizer, group=None, **kw) -> Optimizer:
    """The sharded form of an (unbound) AdamW over `group`, with the same schedule and hyper-parameters. Optimizers
    that are already sharded, already bound to parameters, or of another kind come back unchanged; so does
    everything in a single-rank job."""
    if getattr(opt, "is_sharded", False) or opt.buffers is not None or type(opt) not in (AdamW,) and \
            type(opt).__name__ != "Adam":
        return opt
    if not dist.is_initialized() or dist.get_world_size(group) <= 1:
        return opt
    new = ShardedAdamW(opt._lr, opt.b1, opt.b2, opt.eps, opt.weight_decay, opt.max_grad_norm, group=group, **kw)
    new.step_count = opt.step_count
    return new


class _ShardedBuffersFacade:
    """Gives the trainer the `buffers` attributes it uses (`collect_autograd_grads`, device, names)."""

    def __init__(self, opt: ShardedAdamW):
        self._opt = opt
        self.names, self.params = opt.names, opt.params
        self.device, self.dtype = opt.param_flat.device, opt.param_flat.dtype
        self.param_flat, self.grad_flat = opt.param_flat, opt.grad_flat
        self.total = opt.total

    def collect_autograd_grads(self) -> None:
        self._opt.collect_autograd_grads()

    def zero_grad(self) -> None:
        self._opt.zero_grad()
