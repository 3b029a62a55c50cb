"""Tensor parallelism with sequence-parallel activations on CPU ranks (gloo): the sliced model trains like the whole one."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    from tunix_b200 import optim
    from tunix_b200.common.configs import TrainingConfig
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.parallel import tp as tp_lib
    from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput
    cfg = ModelConfig.tiny_llama().replace(num_layers=2, vocab_size=256, embed_dim=64, hidden_dim=128, num_heads=4,
                                           head_dim=16, num_kv_heads=2)
    model = create_model(cfg, seed=0)
    full = {n: p.detach().clone() for n, p in model.named_parameters()}
    if world > 1:
        tp_lib.apply_tensor_parallel(model, tp_lib.TPContext(device="cpu"))
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, 256, (4, 24), generator=g)
    mask = torch.ones(4, 24)
    mask[1, :7] = 0
    tr = PeftTrainer(model, optim.AdamW(1e-2, weight_decay=0.01, max_grad_norm=0.5),
                     TrainingConfig(eval_every_n_steps=1000, max_steps=3, pbar_description=None))
    tr.train([TrainingInput(toks, mask)] * 3)
    res = {n: p.detach().clone() for n, p in model.named_parameters()}
    torch.save(res, f"{out}.{rank}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return full


def test_tp2_training_matches_single_process(tmp_path):
    base = str(tmp_path / "one")
    _run(0, 1, 0, base)
    mp.spawn(_run, args=(2, 29741, str(tmp_path / "two")), nprocs=2, join=True)
    one = torch.load(base + ".0")
    parts = [torch.load(str(tmp_path / "two") + f".{r}") for r in range(2)]
    for n, w in one.items():
        if any(k in n for k in ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")):
            got = torch.cat([p[n] for p in parts], 0)
        elif any(k in n for k in ("o_proj", "down_proj")):
            got = torch.cat([p[n] for p in parts], 1)
        else:
            assert torch.allclose(parts[0][n], parts[1][n], atol=1e-6), n   # replicated parameters stay in step
            got = parts[0][n]
        assert torch.allclose(got, w, atol=3e-5, rtol=1e-4), (n, (got - w).abs().max())


def _vocab_parallel(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tunix_b200.ops import reference as R
    from tunix_b200.parallel import tp as tp_lib
    tp = tp_lib.TPContext(device="cpu")
    g = torch.Generator().manual_seed(3)                      # the same tensors on every rank
    rows, D, V = 37, 32, 96
    h = torch.randn(rows, D, generator=g).requires_grad_()
    w = (torch.randn(V, D, generator=g) * 0.3)
    t = torch.randint(0, V, (rows,), generator=g)
    t[5] = -1
    gout = torch.randn(rows, generator=g)
    res = {}
    for softcap, temp in ((0.0, 1.0), (5.0, 0.7)):
        ws = w[rank * V // world:(rank + 1) * V // world].clone().requires_grad_()
        lp, ent = tp_lib.vocab_parallel_logprobs(h, ws, t, tp, softcap=softcap, temperature=temp, want_entropy=True, chunk=16)
        (lp * gout).sum().backward()
        wf = w.clone().requires_grad_()
        hf = h.detach().clone().requires_grad_()
        lp_ref, ent_ref = R.lm_head_logprobs_ref(hf, wf, t, softcap=softcap, temperature=temp, want_entropy=True)
        (lp_ref * gout).sum().backward()
        key = f"{softcap}_{temp}"
        res[key] = [float((lp - lp_ref).abs().max()), float((ent - ent_ref).abs().max()),
                    float((h.grad - hf.grad).abs().max()),
                    float((ws.grad - wf.grad[rank * V // world:(rank + 1) * V // world]).abs().max())]
        h.grad = None
    torch.save(res, f"{out}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


def test_vocab_parallel_logprobs_match_full_head(tmp_path):
    mp.spawn(_vocab_parallel, args=(2, 29747, str(tmp_path / "vp")), nprocs=2, join=True)
    for rank in range(2):
        res = torch.load(str(tmp_path / "vp") + f".{rank}")
        for key, errs in res.items():
            assert max(errs) < 2e-4, (rank, key, errs)


def _ckpt(rank, world, port, root, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tunix_b200 import optim
    from tunix_b200.common.configs import TrainingConfig
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.parallel import tp as tp_lib
    from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput
    cfg = ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=128, embed_dim=32, hidden_dim=64, num_heads=2,
                                           head_dim=16, num_kv_heads=2)

    def build(seed):
        m = create_model(cfg, seed=seed)
        return tp_lib.apply_tensor_parallel(m, tp_lib.TPContext(device="cpu"))

    g = torch.Generator().manual_seed(5)
    toks, mask = torch.randint(0, 128, (2, 16), generator=g), torch.ones(2, 16)
    tc = TrainingConfig(eval_every_n_steps=1000, max_steps=2, pbar_description=None, checkpoint_root_directory=root,
                        checkpointing_options={"save_interval_steps": 1, "enable_async_checkpointing": rank == 0})
    tr = PeftTrainer(build(0), optim.AdamW(1e-2, weight_decay=0.0), tc)
    tr.train([TrainingInput(toks, mask)] * 2)                      # every rank calls save(); one of them writes
    trained = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    mu = {n: t.clone() for n, t in tr.optimizer.state_dict()["mu"].items()}
    dist.barrier()
    # a fresh, differently initialised model picks the state up on construction (resume_from_checkpoint_on_init)
    tr2 = PeftTrainer(build(1), optim.AdamW(1e-2, weight_decay=0.0), tc)
    ok = tr2.train_steps == 2
    for n, p in tr2.model.named_parameters():
        ok = ok and torch.equal(p.detach(), trained[n])
    for n, t in tr2.optimizer.state_dict()["mu"].items():
        ok = ok and torch.allclose(t, mu[n])
    torch.save({"ok": bool(ok), "shapes": {n: tuple(p.shape) for n, p in trained.items()}}, f"{out}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


def test_checkpoint_of_a_tp_sliced_model_holds_whole_tensors_and_restores_each_slice(tmp_path):
    root, out = str(tmp_path / "ck"), str(tmp_path / "res")
    mp.spawn(_ckpt, args=(2, 29745, root, out), nprocs=2, join=True)
    res = [torch.load(f"{out}.{r}") for r in range(2)]
    assert all(r["ok"] for r in res)
    from tunix_b200.sft.checkpoint_manager import _load_item
    import json
    saved = _load_item(os.path.join(root, "2", "model_params"))
    q = saved["layers"]["0"]["self_attn"]["q_proj"]["weight"]            # nested by name parts, whole rows
    assert tuple(q.shape) == (32, 32) and res[0]["shapes"]["layers.0.self_attn.q_proj.weight"] == (16, 32)
    assert tuple(saved["layers"]["0"]["mlp"]["down_proj"]["weight"].shape) == (32, 64)
    md = json.load(open(os.path.join(root, "2", "model_params", "_METADATA")))["tree_metadata"]
    assert "('layers', '0', 'self_attn', 'q_proj', 'weight')" in md
    assert sorted(d for d in os.listdir(root) if not d.isdigit()) == []   # no temporary directory left behind


def _run_lora(rank, world, port, out, lora_first):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    from tunix_b200 import lora, optim
    from tunix_b200.common.configs import TrainingConfig
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.parallel import tp as tp_lib
    from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput
    cfg = ModelConfig.tiny_llama().replace(num_layers=2, vocab_size=256, embed_dim=64, hidden_dim=128, num_heads=4,
                                           head_dim=16, num_kv_heads=2)
    model = create_model(cfg, seed=0)
    prov = lora.LoraProvider(rank=4, alpha=8.0)

    def nonzero_b(m):            # a zero B would leave A without gradient in the first step
        g = torch.Generator().manual_seed(11)
        with torch.no_grad():
            for n, p in sorted(m.named_parameters()):
                if n.endswith("lora_b"):
                    p.copy_(torch.randn(p.shape, generator=g) * 0.05)

    if world == 1:
        lora.apply_lora_to_model(model, prov, seed=3)
        nonzero_b(model)
    elif lora_first:
        lora.apply_lora_to_model(model, prov, seed=3)
        nonzero_b(model)
        tp_lib.apply_tensor_parallel(model, tp_lib.TPContext(device="cpu"))
    else:
        tp_lib.apply_tensor_parallel(model, tp_lib.TPContext(device="cpu"))
        lora.apply_lora_to_model(model, prov, seed=3)
        # the same B values as the unsplit model: draw the full matrices, keep this rank's rows of the column-split ones
        g = torch.Generator().manual_seed(11)
        with torch.no_grad():
            for n, p in sorted(model.named_parameters()):
                if n.endswith("lora_b"):
                    col = any(k in n for k in ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj"))
                    full = torch.randn((p.shape[0] * (world if col else 1), p.shape[1]), generator=g) * 0.05
                    p.copy_(full[rank * p.shape[0]:(rank + 1) * p.shape[0]] if col else full)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, 256, (4, 24), generator=g)
    mask = torch.ones(4, 24)
    mask[1, :7] = 0
    tr = PeftTrainer(model, optim.AdamW(1e-2, max_grad_norm=0.5),
                     TrainingConfig(eval_every_n_steps=1000, max_steps=3, pbar_description=None))
    tr.train([TrainingInput(toks, mask)] * 3)
    torch.save({n: p.detach().clone() for n, p in model.named_parameters() if "lora_" in n}, f"{out}.{rank}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _check_lora(one, parts):
    col, row = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj"), ("o_proj", "down_proj")
    assert one and set(one) == set(parts[0])
    for n, w in one.items():
        if n.endswith("lora_b") and any(k in n for k in col):
            got = torch.cat([p[n] for p in parts], 0)
        elif n.endswith("lora_a") and any(k in n for k in row):
            got = torch.cat([p[n] for p in parts], 1)
        else:
            assert torch.allclose(parts[0][n], parts[1][n], atol=1e-6), n
            got = parts[0][n]
        assert torch.allclose(got, w, atol=3e-5, rtol=1e-4), (n, (got - w).abs().max())


def test_tp2_lora_training_matches_single_process(tmp_path):
    """Adapters under tensor parallelism, attached before or after the split: the trained adapters equal the unsplit run."""
    base = str(tmp_path / "one")
    _run_lora(0, 1, 0, base, True)
    one = torch.load(base + ".0")
    for i, lora_first in enumerate((True, False)):
        out = str(tmp_path / f"two{i}")
        mp.spawn(_run_lora, args=(2, 29745 + 2 * i, out, lora_first), nprocs=2, join=True)
        _check_lora(one, [torch.load(out + f".{r}") for r in range(2)])
