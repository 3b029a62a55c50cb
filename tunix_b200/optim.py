"""Optimizers and learning-rate schedules over flat parameter buffers.

The reference builds optimizers from optax (`optax.adamw` + `optax.schedules.*`, optionally chained
with `clip_by_global_norm`; tunix/cli/config.py:210-378) and the trainer applies them inside the
jitted step (tunix/sft/peft_trainer.py:517-548). Here an optimizer owns:

  * one flat buffer of the trainable parameters in their compute dtype (the parameters become views),
  * one flat gradient buffer (`main_grad` views; wgrad GEMMs accumulate into it directly),
  * fp32 master weights (only when the parameters are not fp32) and the moment buffers.

On CUDA every update is one fused kernel launch over the flat buffers (csrc/optim.cu); on CPU the same
math runs in PyTorch. The flat layout is what `parallel/fsdp.py` shards across ranks.
"""
from __future__ import annotations

import math
from typing import Callable, Iterable, Optional, Union

import torch
import torch.nn as nn

Schedule = Callable[[int], float]


# ------------------------------------------------------------------- schedules
def constant_schedule(value: float) -> Schedule:
    return lambda step: float(value)


def linear_schedule(init_value: float, end_value: float, transition_steps: int, transition_begin: int = 0) -> Schedule:
    def f(step):
        if transition_steps <= 0:
            return float(end_value)
        frac = min(max(step - transition_begin, 0) / transition_steps, 1.0)
        return float(init_value + frac * (end_value - init_value))
    return f


def cosine_decay_schedule(init_value: float, decay_steps: int, alpha: float = 0.0) -> Schedule:
    def f(step):
        frac = min(max(step, 0) / max(decay_steps, 1), 1.0)
        cos = 0.5 * (1 + math.cos(math.pi * frac))
        return float(init_value * ((1 - alpha) * cos + alpha))
    return f


def warmup_cosine_decay_schedule(init_value: float, peak_value: float, warmup_steps: int, decay_steps: int,
                                 end_value: float = 0.0) -> Schedule:
    """Linear warm-up to `peak_value`, cosine decay to `end_value` at `decay_steps` (total, incl. warm-up)."""
    def f(step):
        if warmup_steps > 0 and step < warmup_steps:
            return float(init_value + (peak_value - init_value) * step / warmup_steps)
        span = max(decay_steps - warmup_steps, 1)
        frac = min(max(step - warmup_steps, 0) / span, 1.0)
        return float(end_value + (peak_value - end_value) * 0.5 * (1 + math.cos(math.pi * frac)))
    return f


def warmup_constant_schedule(init_value: float, peak_value: float, warmup_steps: int) -> Schedule:
    return lambda step: float(peak_value if step >= warmup_steps or warmup_steps <= 0
                              else init_value + (peak_value - init_value) * step / warmup_steps)


SCHEDULES = {
    "constant_schedule": constant_schedule,
    "linear_schedule": linear_schedule,
    "cosine_decay_schedule": cosine_decay_schedule,
    "warmup_cosine_decay_schedule": warmup_cosine_decay_schedule,
    "warmup_constant_schedule": warmup_constant_schedule,
}


def install_grad_fold_hook(p: nn.Parameter) -> None:
    """A gradient that autograd delivers through `.grad` (an op without a `main_grad` epilogue) is added to the
    parameter's slot of the flat buffer as soon as it has been accumulated, and `.grad` is released: no second
    full-size gradient copy piles up during backward, and an optimizer that reduces a layer's gradients while
    backward still runs finds them in the flat buffer."""
    if getattr(p, "_fold_hook", None) is not None or not hasattr(p, "register_post_accumulate_grad_hook"):
        return

    def fold(param):
        mg = getattr(param, "main_grad", None)
        if mg is not None and param.grad is not None:
            mg.add_(param.grad.to(mg.dtype))
            param.grad = None
            param.grad_added_to_main_grad = True
    p._fold_hook = p.register_post_accumulate_grad_hook(fold)


# ------------------------------------------------------------------ flat buffers
class FlatBuffers:
    """Flat parameter / gradient / state storage for a list of trainable parameters."""

    def __init__(self, named_params: list[tuple[str, nn.Parameter]], grad_dtype: Optional[torch.dtype] = None,
                 align: int = 128, pad_to_multiple: int = 1):
        assert named_params, "no trainable parameters"
        self.names = [n for n, _ in named_params]
        self.params = [p for _, p in named_params]
        dev, dt = self.params[0].device, self.params[0].dtype
        for p in self.params:
            assert p.device == dev and p.dtype == dt, "trainable parameters must share device and dtype"
        self.device, self.dtype = dev, dt
        self.offsets, off = [], 0
        for p in self.params:
            self.offsets.append(off)
            off += (p.numel() + align - 1) // align * align
        total = (off + pad_to_multiple - 1) // pad_to_multiple * pad_to_multiple
        self.total = total
        self.param_flat = torch.zeros(total, dtype=dt, device=dev)
        self.grad_dtype = grad_dtype or (torch.float32 if dt == torch.float32 else torch.bfloat16)
        self.grad_flat = torch.zeros(total, dtype=self.grad_dtype, device=dev)
        with torch.no_grad():
            for p, o in zip(self.params, self.offsets):
                view = self.param_flat[o:o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.main_grad = self.grad_flat[o:o + p.numel()].view(p.shape)
                p.grad_added_to_main_grad = False
                install_grad_fold_hook(p)
        self.master = None if dt == torch.float32 else self.param_flat.float()

    def master_flat(self) -> torch.Tensor:
        return self.param_flat if self.master is None else self.master

    def collect_autograd_grads(self) -> None:
        """Fold gradients that arrived through `.grad` into the flat buffer."""
        for p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(self.grad_dtype))
                p.grad = None

    def zero_grad(self) -> None:
        self.grad_flat.zero_()
        for p in self.params:
            p.grad = None

    def view_of(self, flat: torch.Tensor, i: int) -> torch.Tensor:
        p, o = self.params[i], self.offsets[i]
        return flat[o:o + p.numel()].view(p.shape)


# -------------------------------------------------------------------- optimizers
class Optimizer:
    """Base: learning-rate schedule, global-norm clipping, flat-buffer binding."""

    def __init__(self, learning_rate: Union[float, Schedule], max_grad_norm: Optional[float] = None):
        self._lr = learning_rate if callable(learning_rate) else constant_schedule(learning_rate)
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self.buffers: Optional[FlatBuffers] = None
        self._sumsq = None

    def learning_rate_at(self, step: int) -> float:
        return float(self._lr(step))

    def bind(self, named_params: Iterable[tuple[str, nn.Parameter]], grad_dtype: Optional[torch.dtype] = None,
             pad_to_multiple: int = 1) -> "Optimizer":
        self.buffers = FlatBuffers(list(named_params), grad_dtype, pad_to_multiple=pad_to_multiple)
        self._init_state()
        return self

    def _init_state(self) -> None:
        raise NotImplementedError

    def zero_grad(self) -> None:
        self.buffers.zero_grad()

    def _native(self) -> bool:
        return self.buffers.device.type == "cuda"

    def grad_sumsq(self) -> torch.Tensor:
        """sum(g^2) of the raw accumulated gradients as a device scalar (fp32)."""
        b = self.buffers
        if self._sumsq is None:
            self._sumsq = torch.zeros(1, dtype=torch.float32, device=b.device)
        self._sumsq.zero_()
        if self._native():
            from .ops import kernels as K
            K.sumsq(b.grad_flat, self._sumsq)
        else:
            self._sumsq += b.grad_flat.float().pow(2).sum()
        return self._sumsq

    def step(self, denominator: Union[float, torch.Tensor] = 1.0, sumsq: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Apply one update with grads / denominator. Returns the (pre-clip) global grad norm, a device scalar.

        `sumsq` may be passed in when it was already reduced across ranks. `denominator` may be a one-element
        tensor on the parameters' device: the update kernel then divides by it on the device and the host never
        reads it (the reference trainer likewise keeps the accumulated denominator inside its jitted step,
        tunix/sft/peft_trainer.py:517-548)."""
        b = self.buffers
        b.collect_autograd_grads()
        if sumsq is None:
            sumsq = self.grad_sumsq()
        self.step_count += 1
        lr = self.learning_rate_at(self.step_count - 1)
        if isinstance(denominator, torch.Tensor) and self._native() and self._device_denominator:
            den = denominator.reshape(1).to(torch.float32).clamp_min(1e-8)
            self._apply(lr, 1.0, sumsq, den)
            return sumsq.sqrt() / den
        inv = 1.0 / max(float(denominator), 1e-8)
        self._apply(lr, inv, sumsq)
        return sumsq.sqrt() * inv

    _device_denominator = False   # subclasses whose kernels read the denominator from device memory set this

    def _apply(self, lr: float, grad_scale: float, sumsq: torch.Tensor, denom: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError

    def _clip_scale_cpu(self, grad_scale: float, sumsq: torch.Tensor) -> float:
        scale = grad_scale
        if self.max_grad_norm and self.max_grad_norm > 0:
            norm = float(sumsq.sqrt()) * abs(grad_scale)
            scale *= self.max_grad_norm / max(norm, self.max_grad_norm)
        return scale

    # -- checkpointing: per-parameter views of the flat state
    def state_dict(self) -> dict:
        out = {"step": self.step_count}
        for key, flat in self._state_tensors().items():
            out[key] = {n: self.buffers.view_of(flat, i).detach() for i, n in enumerate(self.buffers.names)}
        return out

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd.get("step", 0))
        for key, flat in self._state_tensors().items():
            if key not in sd:
                continue
            for i, n in enumerate(self.buffers.names):
                if n in sd[key]:
                    self.buffers.view_of(flat, i).copy_(torch.as_tensor(sd[key][n]).to(flat.device, flat.dtype))
        if self.buffers.master is not None and "master" not in sd:
            self.buffers.master.copy_(self.buffers.param_flat.float())

    def sync_master_from_params(self) -> None:
        """Call after parameters were overwritten from outside (checkpoint restore, weight sync)."""
        if self.buffers.master is not None:
            self.buffers.master.copy_(self.buffers.param_flat.float())

    def _state_tensors(self) -> dict:
        return {}


class AdamW(Optimizer):
    """optax.adamw semantics: p -= lr * (m_hat / (sqrt(v_hat) + eps) + weight_decay * p)."""

    def __init__(self, learning_rate: Union[float, Schedule] = 1e-3, b1: float = 0.9, b2: float = 0.999,
                 eps: float = 1e-8, weight_decay: float = 1e-4, max_grad_norm: Optional[float] = None):
        super().__init__(learning_rate, max_grad_norm)
        self.b1, self.b2, self.eps, self.weight_decay = b1, b2, eps, weight_decay

    def _init_state(self) -> None:
        b = self.buffers
        self.m = torch.zeros(b.total, dtype=torch.float32, device=b.device)
        self.v = torch.zeros(b.total, dtype=torch.float32, device=b.device)

    def _state_tensors(self) -> dict:
        d = {"mu": self.m, "nu": self.v}
        if self.buffers.master is not None:
            d["master"] = self.buffers.master
        return d

    _device_denominator = True

    def _apply(self, lr, grad_scale, sumsq, denom=None):
        b = self.buffers
        t = self.step_count
        if self._native():
            from .ops import kernels as K
            K.adamw(b.master_flat(), self.m, self.v, b.grad_flat, b.param_flat if b.master is not None else None,
                    lr=lr, beta1=self.b1, beta2=self.b2, eps=self.eps, weight_decay=self.weight_decay, step=t,
                    grad_scale=grad_scale, max_norm=self.max_grad_norm or 0.0, sumsq_buf=sumsq, denom_buf=denom)
            return
        scale = self._clip_scale_cpu(grad_scale, sumsq)
        with torch.no_grad():
            g = b.grad_flat.float() * scale
            self.m.mul_(self.b1).add_(g, alpha=1 - self.b1)
            self.v.mul_(self.b2).addcmul_(g, g, value=1 - self.b2)
            mhat = self.m / (1 - self.b1 ** t)
            vhat = self.v / (1 - self.b2 ** t)
            p = b.master_flat()
            p.sub_(lr * (mhat / (vhat.sqrt() + self.eps) + self.weight_decay * p))
            if b.master is not None:
                b.param_flat.copy_(p.to(b.dtype))


class Adam(AdamW):
    def __init__(self, learning_rate=1e-3, b1=0.9, b2=0.999, eps=1e-8, max_grad_norm=None):
        super().__init__(learning_rate, b1, b2, eps, 0.0, max_grad_norm)


class SGD(Optimizer):
    def __init__(self, learning_rate=1e-2, momentum: float = 0.0, weight_decay: float = 0.0, max_grad_norm=None):
        super().__init__(learning_rate, max_grad_norm)
        self.momentum, self.weight_decay = momentum, weight_decay

    def _init_state(self) -> None:
        b = self.buffers
        self.mom = torch.zeros(b.total, dtype=torch.float32, device=b.device) if self.momentum else None

    def _state_tensors(self) -> dict:
        d = {} if self.mom is None else {"trace": self.mom}
        if self.buffers.master is not None:
            d["master"] = self.buffers.master
        return d

    def _apply(self, lr, grad_scale, sumsq, denom=None):
        b = self.buffers
        scale = self._clip_scale_cpu(grad_scale, sumsq) if (self.max_grad_norm or not self._native()) else grad_scale
        if self._native():
            from .ops import kernels as K
            K.sgd(b.master_flat(), self.mom, b.grad_flat, b.param_flat if b.master is not None else None, lr=lr,
                  momentum=self.momentum, weight_decay=self.weight_decay, scale=scale)
            return
        with torch.no_grad():
            p = b.master_flat()
            g = b.grad_flat.float() * scale + self.weight_decay * p
            if self.mom is not None:
                self.mom.mul_(self.momentum).add_(g)
                g = self.mom
            p.sub_(lr * g)
            if b.master is not None:
                b.param_flat.copy_(p.to(b.dtype))


OPTIMIZERS = {"adamw": AdamW, "adam": Adam, "sgd": SGD}


def create_optimizer(opt_type: str = "adamw", learning_rate: Union[float, Schedule, None] = None,
                     schedule_type: Optional[str] = None, schedule_kwargs: Optional[dict] = None,
                     max_grad_norm: Optional[float] = None, **kwargs) -> Optimizer:
    """Factory used by the CLI: `opt_type` + optional `schedule_type` with kwargs filtered by signature."""
    import inspect
    if opt_type not in OPTIMIZERS:
        raise ValueError(f"unknown optimizer {opt_type!r}; known: {sorted(OPTIMIZERS)}")
    if schedule_type:
        if schedule_type not in SCHEDULES:
            raise ValueError(f"unknown schedule {schedule_type!r}; known: {sorted(SCHEDULES)}")
        fn = SCHEDULES[schedule_type]
        allowed = inspect.signature(fn).parameters
        lr = fn(**{k: v for k, v in (schedule_kwargs or {}).items() if k in allowed})
    else:
        lr = learning_rate if learning_rate is not None else 1e-3
    cls = OPTIMIZERS[opt_type]
    allowed = inspect.signature(cls.__init__).parameters
    kw = {k: v for k, v in kwargs.items() if k in allowed}
    return cls(learning_rate=lr, max_grad_norm=max_grad_norm, **kw)
