"""`python -m tunix_b200.cli.peft_main base_config.yaml key=value ...` — SFT / LoRA / QLoRA
(tunix/cli/peft_main.py:36-112)."""
from __future__ import annotations

import os
import sys

import torch

from ..common.configs import CheckpointingOptions, MetricsLoggerOptions, ProfilerOptions, TrainingConfig
from ..sft.peft_trainer import PeftTrainer
from . import config as config_lib
from .utils import data as data_lib, model as model_lib


def training_config_from(d: dict, cls=TrainingConfig, **extra):
    d = dict(d)
    ml = d.pop("metrics_logging_options", None)
    po = d.pop("profiler_options", None)
    d.pop("perf_metrics_options", None)
    ck = d.pop("checkpointing_options", None)
    known = {f for f in cls.__dataclass_fields__}
    kw = {k: v for k, v in d.items() if k in known}
    if "data_sharding_axis" in kw:
        kw["data_sharding_axis"] = tuple(kw["data_sharding_axis"])
    return cls(**kw, metrics_logging_options=MetricsLoggerOptions(**ml) if ml else None,
               profiler_options=ProfilerOptions(**po) if po and po.get("log_dir") else None,
               checkpointing_options=CheckpointingOptions.from_dict(ck) if ck else None, **extra)


def init_distributed():
    import torch.distributed as dist
    if "RANK" in os.environ and not dist.is_initialized():
        use_cuda = torch.cuda.is_available()
        if use_cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl" if use_cuda else "gloo")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if torch.cuda.is_available() else torch.device("cpu")
    return dev


def run_peft_trainer(hp: config_lib.HyperParameters):
    """The mesh of `model_config.mesh` picks the parallel strategy (`parallel/strategy.py`): an `fsdp` axis ->
    sharded optimizer (or, with `model_config.shard_weights`, weights sharded too and gathered inside the GEMMs),
    a `tp` axis -> tensor parallelism, both -> tensor-parallel groups that are data-parallel replicas."""
    from ..parallel import strategy
    dev = init_distributed()
    mesh = hp.create_mesh()
    model = model_lib.create_model(hp["model_config"], device=dev)
    tok = model_lib.create_tokenizer(hp["tokenizer_config"])
    tc = training_config_from(hp["training_config"])
    opt, plan = strategy.apply_parallelism(model, hp.create_optimizer(), mesh,
                                           shard_weights=bool(hp["model_config"].get("shard_weights", False)), device=dev)
    trainer = PeftTrainer(model, opt, tc)
    trainer.parallel_plan = plan
    train_ds, eval_ds = data_lib.create_datasets(hp, tok, model.config.vocab_size)
    trainer.train(train_ds, eval_ds)
    return trainer


def main(argv=None):
    hp = config_lib.HyperParameters(sys.argv if argv is None else argv)
    return run_peft_trainer(hp)


if __name__ == "__main__":
    main()
