"""Compare this framework's forward pass with the Hugging Face implementation on the same checkpoint
(the job of the reference's scripts/forward_pass_logit_checker.py).

    python -m tunix_b200.models.logit_checker --model-path /path/to/hf_checkpoint [--prompt "..."] [--tokens 64]
           [--device cuda] [--dtype float32] [--atol 1e-3]

Both models read the same safetensors; the prompt is tokenised with the checkpoint's tokenizer when there is one,
else random token ids are used. Reports the largest absolute and relative logit differences, the mean KL
divergence between the two next-token distributions and the top-1 agreement, and exits non-zero when the largest
absolute difference exceeds `--atol`."""
from __future__ import annotations

import argparse
import json
import sys
from typing import Optional

import torch


def compare_logits(ours: torch.Tensor, ref: torch.Tensor) -> dict:
    a, b = ours.float(), ref.float()
    diff = (a - b).abs()
    la, lb = torch.log_softmax(a, -1), torch.log_softmax(b, -1)
    return {"max_abs_diff": float(diff.max()), "mean_abs_diff": float(diff.mean()),
            "max_rel_diff": float((diff / b.abs().clamp_min(1e-3)).max()),
            "kl_ref_to_ours": float((lb.exp() * (lb - la)).sum(-1).mean()),
            "top1_agreement": float((a.argmax(-1) == b.argmax(-1)).float().mean())}


def check(model_path: str, prompt: Optional[str] = None, tokens: int = 64, device: str = "cpu",
          dtype: torch.dtype = torch.float32, seed: int = 0, config_overrides: Optional[dict] = None) -> dict:
    import transformers
    from .hf_config import config_from_hf
    from .safetensors_loader import load_safetensors_into
    from .transformer import create_model
    cfg = config_from_hf(model_path, dtype=dtype, **(config_overrides or {}))
    ids = None
    if prompt is not None:
        try:
            tok = transformers.AutoTokenizer.from_pretrained(model_path)
            ids = torch.tensor([tok(prompt)["input_ids"]])
        except Exception as e:                              # no tokenizer files beside the weights
            print(f"no tokenizer ({type(e).__name__}); using random token ids", file=sys.stderr)
    if ids is None:
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(0, cfg.vocab_size, (2, min(tokens, cfg.max_position)), generator=g)
    hf = transformers.AutoModelForCausalLM.from_pretrained(model_path, torch_dtype=dtype, attn_implementation="eager").eval().to(device)
    ours = create_model(cfg, device=torch.device(device), seed=seed)
    load_safetensors_into(ours, model_path)
    ours.eval()
    ids = ids.to(device)
    with torch.no_grad():
        ref = hf(ids).logits
        got = ours(ids)[0]
    out = compare_logits(got, ref)
    out.update(family=cfg.family, tokens=int(ids.numel()), dtype=str(dtype).replace("torch.", ""), device=device)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model-path", required=True)
    ap.add_argument("--prompt", default=None)
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16", "float16"])
    ap.add_argument("--atol", type=float, default=1e-3)
    a = ap.parse_args(argv)
    out = check(a.model_path, a.prompt, a.tokens, a.device, getattr(torch, a.dtype))
    out["ok"] = out["max_abs_diff"] <= a.atol
    print(json.dumps(out))
    return 0 if out["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
