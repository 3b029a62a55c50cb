"""Vision tower, soft-token splice and bidirectional image spans (CPU, tiny sizes)."""
import torch

from tunix_b200.models import vision as V
from tunix_b200.testing.common import ToyTransformer


def test_tower_shapes_and_pooling():
    cfg = V.VisionConfig.tiny()
    tower = V.VisionTower(cfg)
    imgs = torch.randn(2, 3, 32, 32, 3)
    out = tower(imgs)
    assert out.shape == (2, 3, 4, 64)
    p = tower.patchify(torch.arange(32 * 32 * 3, dtype=torch.float32).view(1, 32, 32, 3))
    assert p.shape == (1, 16, 8 * 8 * 3) and p[0, 1, 0] == 8 * 3          # second patch starts 8 pixels to the right


def test_merge_places_soft_tokens_in_order():
    text = torch.zeros(2, 6, 3)
    vis = torch.arange(2 * 1 * 2 * 3, dtype=torch.float32).view(2, 1, 2, 3) + 1
    mask = torch.tensor([[0, 1, 1, 0, 0, 0], [0, 0, 0, 0, 0, 0]], dtype=torch.bool)
    out = V.merge_embeddings(text, vis, mask)
    assert torch.equal(out[0, 1], vis[0, 0, 0]) and torch.equal(out[0, 2], vis[0, 0, 1]) and float(out[1].abs().sum()) == 0
    spans = V.image_span_ids(torch.tensor([[5, 9, 9, 9, 9, 7]]), 9, 2)
    assert spans.tolist() == [[0, 1, 1, 2, 2, 0]]


def test_multimodal_forward_backward_and_bidirectional_mask():
    lm = ToyTransformer(vocab_size=128, num_layers=1)
    vc = V.VisionConfig.tiny(image_token_id=100)
    mm = V.Gemma3Multimodal(lm, vc)
    toks = torch.tensor([[1, 100, 100, 100, 100, 7, 8, 9]])
    imgs = torch.randn(1, 1, 32, 32, 3)
    logits, _ = mm(toks, images=imgs)
    assert logits.shape == (1, 8, 128)
    logits.float().logsumexp(-1).sum().backward()
    assert mm.vision_tower.patch_embed.weight.grad is not None and mm.projector.proj.grad.abs().sum() > 0
    # the first image token sees the later ones (bidirectional span): changing the image changes position 1's output
    with torch.no_grad():
        a = mm(toks, images=imgs)[0]
        imgs2 = imgs.clone()
        imgs2[0, 0, 16:, 16:] += 1.0                   # only the last patch row/col -> only the last soft tokens differ
        b = mm(toks, images=imgs2)[0]
    assert not torch.allclose(a[0, 1], b[0, 1])
    text_only = mm(toks[:, 5:])[0]
    assert text_only.shape == (1, 3, 128)
